"""warp34_b200: B200 (sm_100a) implementation of the TQ4 paged-KV hot path.

Layout of the package:
  csrc/      CUDA kernels + C ABI (include/warp34_b200.h), host page manager (include/warp34_host.h)
  build.py   in-tree nvcc / g++ build of lib/libwarp34_b200.so and lib/libwarp34_host.so
  ffi.py     ctypes bindings of both ABIs
  kv.py      host-side mirror of the reference's KvPool / request page state / step metadata
  synth.py   seeded synthetic workloads of the benchmark configurations
  sharding.py  how batches, KV heads and pages are cut across GPUs
"""
from . import ffi  # noqa: F401

__all__ = ["ffi"]
