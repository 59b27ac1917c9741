"""``import tbvcoll`` — the reference's module name (step4/tbvcoll.py), re-exporting the
B200 build's handle so that scripts written against the reference run unchanged."""
from libtbvcoll_b200.tbvcoll import *  # noqa: F401,F403
from libtbvcoll_b200.tbvcoll import Comm, init, init_n, all_reduce, synchronize, is_async, err, rails, hist, raw_fn, cap, stats5, stats4, stats3, stats, fini, comm  # noqa: F401
