"""B200-native backend for the Gaudi MME compute reference (CPUCalculator): GEMM, batched GEMM and
convolution fwd / dedx / dedw over bf16, fp32, fp8_143 and fp8_152 with fp32 accumulation and a
rounded output cast, as hand-written sm_100a kernels behind a C ABI (include/mme_b200.h)."""
from . import abi  # noqa: F401
from .calculator import Calculator, DeviceBuffer, MmeError  # noqa: F401
