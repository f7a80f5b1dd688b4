"""B200-native Solid GPU core behind Ocean's operator interface.

`solid_b200._lib`   ctypes binding of the C-ABI library (lib/libsolid_core_gpu.so)
`solid_b200.Tensor` device tensor views (dtype, sizes, byte strides, byte order)
`solid_b200.ops`    operations with Ocean's names (add, scale, sqrt, sum, norm, copy, ...)
`solid_b200.shard`  leading-axis sharding over the GPUs of one node
"""
from . import dtypes, oplist            # noqa: F401
from .tensor import Tensor              # noqa: F401
from . import ops                       # noqa: F401
