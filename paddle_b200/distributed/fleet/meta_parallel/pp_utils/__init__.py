"""Point-to-point helpers of the pipeline schedules (fleet/meta_parallel/pp_utils/)."""
from . import p2p_communication  # noqa: F401
