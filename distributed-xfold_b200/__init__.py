"""B200-native (sm_100a) implementation of the tensor-parallel Pairformer trunk and diffusion
transformer hot path behind the reference's module API.  The directory name carries a hyphen, so
import it through ``__graft_entry__.load_package()`` (registers it as ``distributed_xfold_b200``).
"""
from . import _cabi  # noqa: F401

__all__ = ["_cabi", "ops"]
