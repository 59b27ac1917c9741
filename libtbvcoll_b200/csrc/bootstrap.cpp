// bootstrap.cpp — TCP star rendezvous + unix-socket fd passing (see bootstrap.h).
#include "bootstrap.h"

#include <arpa/inet.h>
#include <errno.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <stdio.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <time.h>
#include <unistd.h>

namespace tbv {

static double now_s() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return ts.tv_sec + ts.tv_nsec * 1e-9;
}

// Full write / full read with a deadline; 0 on success.
static int write_all(int fd, const void* buf, size_t n, double deadline) {
  const char* p = static_cast<const char*>(buf);
  while (n) {
    pollfd pf{fd, POLLOUT, 0};
    double left = deadline - now_s();
    if (left <= 0) return -1;
    int pr = poll(&pf, 1, int(left * 1000) + 1);
    if (pr < 0 && errno == EINTR) continue;
    if (pr <= 0) return -1;
    ssize_t k = ::send(fd, p, n, MSG_NOSIGNAL);
    if (k < 0) {
      if (errno == EINTR || errno == EAGAIN) continue;
      return -1;
    }
    p += k;
    n -= size_t(k);
  }
  return 0;
}
static int read_all(int fd, void* buf, size_t n, double deadline) {
  char* p = static_cast<char*>(buf);
  while (n) {
    pollfd pf{fd, POLLIN, 0};
    double left = deadline - now_s();
    if (left <= 0) return -1;
    int pr = poll(&pf, 1, int(left * 1000) + 1);
    if (pr < 0 && errno == EINTR) continue;
    if (pr <= 0) return -1;
    ssize_t k = ::recv(fd, p, n, 0);
    if (k == 0) return -1;  // peer closed
    if (k < 0) {
      if (errno == EINTR || errno == EAGAIN) continue;
      return -1;
    }
    p += k;
    n -= size_t(k);
  }
  return 0;
}

Bootstrap::~Bootstrap() { close_all(); }

void Bootstrap::close_all() {
  for (int& s : socks_) {
    if (s >= 0) ::close(s);
    s = -1;
  }
  if (listen_fd_ >= 0) ::close(listen_fd_);
  if (uds_fd_ >= 0) ::close(uds_fd_);
  listen_fd_ = uds_fd_ = -1;
}

static void uds_name(sockaddr_un* a, socklen_t* len, int port, int rank) {
  memset(a, 0, sizeof(*a));
  a->sun_family = AF_UNIX;
  // abstract namespace: sun_path[0] == 0, no file to clean up
  int n = snprintf(a->sun_path + 1, sizeof(a->sun_path) - 2, "tbvcoll.%d.%d", port, rank);
  *len = socklen_t(offsetof(sockaddr_un, sun_path) + 1 + n);
}

int Bootstrap::init(int rank, int world, const char* ip, int port, double timeout_s) {
  rank_ = rank;
  world_ = world;
  port_ = port;
  timeout_s_ = timeout_s;
  socks_.assign(world, -1);
  if (world == 1) return 0;
  const double deadline = now_s() + timeout_s;
  const char* host = (ip && *ip) ? ip : "127.0.0.1";

  // fd-passing listener first, so that it exists before anyone passes the barrier
  uds_fd_ = ::socket(AF_UNIX, SOCK_STREAM, 0);
  if (uds_fd_ < 0) { err_ = "socket(AF_UNIX)"; return -1; }
  sockaddr_un ua; socklen_t ulen;
  uds_name(&ua, &ulen, port, rank);
  if (::bind(uds_fd_, reinterpret_cast<sockaddr*>(&ua), ulen) != 0 || ::listen(uds_fd_, 64) != 0) {
    err_ = std::string("bind/listen unix socket: ") + strerror(errno);
    return -1;
  }

  sockaddr_in sa{};
  sa.sin_family = AF_INET;
  sa.sin_port = htons(uint16_t(port));
  if (rank == 0) {
    listen_fd_ = ::socket(AF_INET, SOCK_STREAM, 0);
    int one = 1;
    setsockopt(listen_fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    sa.sin_addr.s_addr = htonl(INADDR_ANY);
    if (::bind(listen_fd_, reinterpret_cast<sockaddr*>(&sa), sizeof(sa)) != 0 ||
        ::listen(listen_fd_, 64) != 0) {
      err_ = std::string("bind/listen tcp: ") + strerror(errno);
      return -1;
    }
    for (int got = 0; got < world - 1;) {
      pollfd pf{listen_fd_, POLLIN, 0};
      double left = deadline - now_s();
      if (left <= 0 || poll(&pf, 1, int(left * 1000) + 1) <= 0) {
        err_ = "timed out waiting for peers to connect";
        return -1;
      }
      int s = ::accept(listen_fd_, nullptr, nullptr);
      if (s < 0) continue;
      int one2 = 1;
      setsockopt(s, IPPROTO_TCP, TCP_NODELAY, &one2, sizeof(one2));
      int hello[2] = {0, 0};
      if (read_all(s, hello, sizeof(hello), deadline) != 0 || hello[0] <= 0 || hello[0] >= world ||
          hello[1] != world || socks_[hello[0]] >= 0) {
        ::close(s);  // a stranger, a duplicate, or a peer that disagrees on the world size
        if (hello[1] != world && hello[0] > 0) { err_ = "peer disagrees on world size"; return -1; }
        continue;
      }
      socks_[hello[0]] = s;
      got++;
    }
  } else {
    if (inet_pton(AF_INET, host, &sa.sin_addr) != 1) { err_ = "bad peer ip"; return -1; }
    int s = -1;
    while (true) {
      s = ::socket(AF_INET, SOCK_STREAM, 0);
      if (::connect(s, reinterpret_cast<sockaddr*>(&sa), sizeof(sa)) == 0) break;
      ::close(s);
      s = -1;
      if (now_s() > deadline) { err_ = "timed out connecting to rank 0"; return -1; }
      usleep(50 * 1000);
    }
    int one = 1;
    setsockopt(s, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    int hello[2] = {rank, world};
    if (write_all(s, hello, sizeof(hello), deadline) != 0) { err_ = "hello failed"; return -1; }
    socks_[0] = s;
  }
  return barrier();
}

int Bootstrap::allgather(const void* mine, void* all, size_t each) {
  char* out = static_cast<char*>(all);
  memcpy(out + size_t(rank_) * each, mine, each);
  if (world_ == 1) return 0;
  const double deadline = now_s() + timeout_s_;
  if (rank_ == 0) {
    for (int r = 1; r < world_; r++)
      if (read_all(socks_[r], out + size_t(r) * each, each, deadline) != 0) { err_ = "allgather: recv"; return -1; }
    for (int r = 1; r < world_; r++)
      if (write_all(socks_[r], out, each * world_, deadline) != 0) { err_ = "allgather: send"; return -1; }
  } else {
    if (write_all(socks_[0], mine, each, deadline) != 0) { err_ = "allgather: send"; return -1; }
    if (read_all(socks_[0], out, each * world_, deadline) != 0) { err_ = "allgather: recv"; return -1; }
  }
  return 0;
}

int Bootstrap::barrier() {
  char b = 'S';
  std::vector<char> all(world_);
  return allgather(&b, all.data(), 1);
}

int Bootstrap::send_fd_to(int peer, int tag, int fd) {
  int s = ::socket(AF_UNIX, SOCK_STREAM, 0);
  if (s < 0) return -1;
  sockaddr_un ua; socklen_t ulen;
  uds_name(&ua, &ulen, port_, peer);
  if (::connect(s, reinterpret_cast<sockaddr*>(&ua), ulen) != 0) { ::close(s); return -1; }
  int hdr[2] = {rank_, tag};
  iovec iov{hdr, sizeof(hdr)};
  alignas(cmsghdr) char cbuf[CMSG_SPACE(sizeof(int))];
  memset(cbuf, 0, sizeof(cbuf));
  msghdr msg{};
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = cbuf;
  msg.msg_controllen = sizeof(cbuf);
  cmsghdr* cm = CMSG_FIRSTHDR(&msg);
  cm->cmsg_level = SOL_SOCKET;
  cm->cmsg_type = SCM_RIGHTS;
  cm->cmsg_len = CMSG_LEN(sizeof(int));
  memcpy(CMSG_DATA(cm), &fd, sizeof(int));
  ssize_t k = ::sendmsg(s, &msg, MSG_NOSIGNAL);
  ::close(s);
  return k == ssize_t(sizeof(hdr)) ? 0 : -1;
}

int Bootstrap::recv_fd(int* src, int* tag, int* fd) {
  pollfd pf{uds_fd_, POLLIN, 0};
  if (poll(&pf, 1, int(timeout_s_ * 1000)) <= 0) return -1;
  int s = ::accept(uds_fd_, nullptr, nullptr);
  if (s < 0) return -1;
  int hdr[2] = {-1, -1};
  iovec iov{hdr, sizeof(hdr)};
  alignas(cmsghdr) char cbuf[CMSG_SPACE(sizeof(int))];
  msghdr msg{};
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = cbuf;
  msg.msg_controllen = sizeof(cbuf);
  pollfd pr{s, POLLIN, 0};
  if (poll(&pr, 1, int(timeout_s_ * 1000)) <= 0) { ::close(s); return -1; }
  ssize_t k = ::recvmsg(s, &msg, 0);
  ::close(s);
  if (k != ssize_t(sizeof(hdr))) return -1;
  cmsghdr* cm = CMSG_FIRSTHDR(&msg);
  if (!cm || cm->cmsg_level != SOL_SOCKET || cm->cmsg_type != SCM_RIGHTS) return -1;
  memcpy(fd, CMSG_DATA(cm), sizeof(int));
  *src = hdr[0];
  *tag = hdr[1];
  return 0;
}

int Bootstrap::allgather_fd(int myfd, std::vector<int>* fds_out) {
  fds_out->assign(world_, -1);
  (*fds_out)[rank_] = myfd;
  if (world_ == 1) return 0;
  if (barrier() != 0) return -1;
  // connect() to a listening unix socket completes from the backlog without an
  // accept(), so "send to everyone, then receive from everyone" cannot deadlock.
  for (int p = 0; p < world_; p++)
    if (p != rank_ && send_fd_to(p, 1, myfd) != 0) { err_ = "fd send failed"; return -1; }
  for (int i = 0; i < world_ - 1; i++) {
    int src, tag, fd;
    if (recv_fd(&src, &tag, &fd) != 0 || src < 0 || src >= world_ || tag != 1 || (*fds_out)[src] >= 0) {
      err_ = "fd receive failed";
      return -1;
    }
    (*fds_out)[src] = fd;
  }
  return barrier();
}

int Bootstrap::broadcast_fd(int root, int myfd, int* fd_out) {
  *fd_out = myfd;
  if (world_ == 1) return 0;
  if (barrier() != 0) return -1;
  if (rank_ == root) {
    for (int p = 0; p < world_; p++)
      if (p != rank_ && send_fd_to(p, 2, myfd) != 0) { err_ = "fd broadcast send failed"; return -1; }
  } else {
    int src, tag, fd;
    if (recv_fd(&src, &tag, &fd) != 0 || src != root || tag != 2) { err_ = "fd broadcast receive failed"; return -1; }
    *fd_out = fd;
  }
  return barrier();
}

}  // namespace tbv
