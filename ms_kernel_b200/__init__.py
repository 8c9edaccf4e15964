"""B200-native MSAQ-signed decode path: weight-only GEMV, KV flash-decode,
KV append with Hadamard rotation.

`ms_kernel_b200.ops` mirrors the reference's `ms_lib/ops.py`; importing it loads
the compiled `ms_cuda` operator module (torch.ops.msaq.*).  The kernels exist
only as CUDA for sm_100a; nothing here falls back to PyTorch or the CPU.
"""

__version__ = "1.0"
