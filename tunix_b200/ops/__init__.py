"""Hot ops: sm_100a kernels with autograd glue (`functional`), raw launchers (`kernels`) and
the PyTorch oracle (`ref`)."""
from . import functional, ref  # noqa: F401
