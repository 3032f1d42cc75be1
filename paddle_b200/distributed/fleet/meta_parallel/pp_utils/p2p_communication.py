"""Re-export of the stage-to-stage transport used by the schedules
(fleet/meta_parallel/pp_utils/p2p_communication.py: ``SendRecvMeta`` :52, ``P2pHelper`` :573)."""
from ..pipeline_parallel import P2pHelper, SendRecvMeta  # noqa: F401
