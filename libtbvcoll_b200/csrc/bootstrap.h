// bootstrap.h — out-of-band rendezvous between the ranks of one node.
//
// Role of the reference's single TCP socket that carries the QP/rkey/addr/GID blob
// and a 1-byte barrier (step4/libtbvcoll.cpp:64, 371-385, 403), generalised to N
// ranks: rank 0 listens, everybody else connects (with retries), and rank 0 relays.
// File descriptors (CUDA VMM shareable handles) travel over abstract unix sockets
// with SCM_RIGHTS.
#pragma once
#include <stddef.h>

#include <string>
#include <vector>

namespace tbv {

class Bootstrap {
 public:
  Bootstrap() = default;
  ~Bootstrap();
  Bootstrap(const Bootstrap&) = delete;
  Bootstrap& operator=(const Bootstrap&) = delete;

  // Returns 0 on success.  timeout_s bounds the whole rendezvous (a peer that never
  // shows up makes init fail instead of blocking for ever).
  int init(int rank, int world, const char* ip, int port, double timeout_s);
  // all[r*each .. (r+1)*each) = rank r's `mine`.
  int allgather(const void* mine, void* all, size_t each);
  int barrier();
  // Every rank contributes one fd; fds_out[r] is a local duplicate of rank r's fd
  // (fds_out[rank] == myfd, not duplicated).
  int allgather_fd(int myfd, std::vector<int>* fds_out);
  // Rank `root` contributes one fd, everyone else receives a duplicate.
  int broadcast_fd(int root, int myfd, int* fd_out);
  void close_all();
  const std::string& error() const { return err_; }

 private:
  int send_fd_to(int peer, int tag, int fd);
  int recv_fd(int* src, int* tag, int* fd);
  int rank_ = 0, world_ = 1, port_ = 0;
  double timeout_s_ = 30.0;
  int listen_fd_ = -1;          // rank 0 TCP listener
  std::vector<int> socks_;      // rank 0: socks_[r]; others: socks_[0]
  int uds_fd_ = -1;             // abstract unix listener for fd passing
  std::string err_;
};

}  // namespace tbv
