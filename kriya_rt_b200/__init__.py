"""B200-native backend for KriyaRT's paged KV-cache hot path.

The package is a thin host-side mirror of the reference's interfaces for this path:

* ``kriya_rt_b200.kv.PagedKvCacheManager`` - the `kriya-kv` manager API
  (crates/kriya-kv/src/bsr_paged.rs) over the compiled C++ bookkeeping library;
* ``kriya_rt_b200.executor.CudaExecutor`` - the attention / KV ops of ``MetalExecutor``
  (crates/kriya-backend-metal/src/encoder.rs) over ``libkriya_cuda.so``.

All compute happens in hand-written sm_100a CUDA kernels behind a C ABI (``include/*.h``).
There is no CPU fallback: if the native libraries are missing, imports of the submodules fail.
"""
__version__ = "0.1.0"
