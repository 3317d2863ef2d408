"""B200-native provider for Trinity Lowering's CUDA path (host-side mirror of the reference's
``trinity_lowering`` Python package; the kernels live behind ``include/trinity_sm100.h``)."""
from . import kernels  # noqa: F401
