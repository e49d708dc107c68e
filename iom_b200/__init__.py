"""iom_b200: B200 (sm_100a) device tensor-op backend for IOM's backend contract.

The package holds the CUDA kernels and their C ABI (csrc/, libiom_b200.so) and
a host-side mirror of the reference's Device / Tensor / DeviceOps interface.
Importing the metadata classes needs neither torch nor a GPU; creating a device
does.
"""
from .tensor import DataType, TensorSpec, TensorView, leaf_bits, plane_slot

__all__ = ["DataType", "TensorSpec", "TensorView", "leaf_bits", "plane_slot",
           "make_b200_device", "DeviceMemoryConfig", "QueueConfig"]


def __getattr__(name):
    if name in ("make_b200_device", "DeviceMemoryConfig", "QueueConfig", "B200Device",
                "B200Queue", "RawWorkspace", "RawWorkspaceView", "UnsupportedOperation"):
        from . import device
        return getattr(device, name)
    raise AttributeError(name)
