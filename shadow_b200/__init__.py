"""shadow_b200: B200 (sm_100a) kernels for Shadow's tensor-operator hot path.

* ``capi``       - ctypes binding of the kernel C ABI (``include/sb200.h``, ``lib/libsb200.so``).
* ``functional`` - operator-level calls on CUDA tensors already resident in HBM.
* ``netapi``     - ctypes binding of the Network C adapter over the C++ host library
                   (``lib/libshadow_b200.so``): the Shadow Operator/Kernel/Blob/Workspace API with
                   the six GPU kernel classes registered behind it.
* ``sharded``    - dim-0 sharding of the operators over the ranks of a torch.distributed job.

There is no CPU fallback anywhere in the package: a missing compiled library raises.
"""
import os

PACKAGE_DIR = os.path.dirname(os.path.abspath(__file__))
KERNEL_LIB = os.path.join(PACKAGE_DIR, "lib", "libsb200.so")
HOST_LIB = os.path.join(PACKAGE_DIR, "lib", "libshadow_b200.so")


def host_library():
    """NetLibrary over the product's C++ host library (raises if it has not been built)."""
    from .netapi import NetLibrary
    if not os.path.exists(HOST_LIB):
        raise ImportError("host library %s is missing: run `python -m shadow_b200.build`" % HOST_LIB)
    return NetLibrary(HOST_LIB, "sb200net_")
