"""torch_projectors_b200 -- B200-native (sm_100a) Fourier-slice operators with the public
API of warpem/torch-projectors.

Importing the package loads ``libb200proj.so`` (hand-written CUDA kernels behind a C ABI,
``include/b200proj.h``) and ``_C.so`` (the C++ operator layer over it, ``csrc/torch_binding.cpp``),
which defines the eight raw operators under ``torch.ops.torch_projectors_b200`` for CUDA tensors.  There is no CPU, MPS or Triton
path: if the library cannot be loaded the import fails, and CPU tensors are rejected by
the dispatcher.

(reference loader: torch_projectors/__init__.py:8-30)
"""
from . import _abi

_abi.load()          # fail loudly at import time if the CUDA library is missing

from . import ops  # noqa: E402  (registers the raw operators)
from .ops import (  # noqa: E402
    backproject_2d_forw,
    backproject_2d_to_3d_accumulate_,
    backproject_2d_to_3d_accumulate_interleaved_,
    fold_backprojection_accumulator,
    fold_backprojection_accumulator_normalized,
    project_3d_to_2d_forw_packed,
    unpack_projections,
    new_backprojection_accumulator,
    plane_locality_order,
    set_pose_order_thresholds,
    set_save_derivatives,
    backproject_2d_to_3d_back,
    backproject_2d_to_3d_forw,
    project_2d_back,
    project_2d_forw,
    project_3d_to_2d_back,
    project_3d_to_2d_forw,
)
from . import sharding  # noqa: E402
from . import streaming  # noqa: E402
from . import prep  # noqa: E402
from .streaming import backproject_2d_to_3d_from_host, project_3d_to_2d_to_host  # noqa: E402

__version__ = "0.3.0"

__all__ = [
    "project_2d_forw", "project_2d_back", "project_3d_to_2d_forw", "project_3d_to_2d_back",
    "backproject_2d_forw", "backproject_2d_to_3d_forw", "backproject_2d_to_3d_back",
    "backproject_2d_to_3d_accumulate_", "backproject_2d_to_3d_accumulate_interleaved_",
    "new_backprojection_accumulator", "fold_backprojection_accumulator", "plane_locality_order",
    "set_pose_order_thresholds", "set_save_derivatives", "fold_backprojection_accumulator_normalized", "project_3d_to_2d_forw_packed",
    "unpack_projections", "sharding", "streaming", "prep",
    "project_3d_to_2d_to_host", "backproject_2d_to_3d_from_host",
]
