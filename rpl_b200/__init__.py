"""rpl_b200: the INT8 quantized-inference path of RPL on B200 (sm_100a).

The product is the shared library ``rpl_b200/lib/librpl.so`` (C ABI in
``include/rpl_b200.h``); the modules here bind it:

``build``    compiles the library in-tree with nvcc / gcc
``capi``     ctypes signatures of every exported function, struct mirrors
``device``   the ``rplb_*`` device-level entry points over torch CUDA tensors
``sharded``  column-parallel quantized Linear across one process per GPU,
             host-buffer pipeline

Nothing is imported eagerly: ``import rpl_b200`` works without torch or a built
library; ``rpl_b200.capi.load()`` fails loudly when the library is missing.
"""

__all__ = ["build", "capi", "device", "sharded"]
