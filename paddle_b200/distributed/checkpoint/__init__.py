"""``paddle.distributed.checkpoint``: sharded save / load with re-partitioning on load."""
from .load_state_dict import CheckpointCorruptError, load_merged_state_dict, load_state_dict  # noqa: F401
from .metadata import LocalTensorIndex, LocalTensorMetadata, Metadata  # noqa: F401
from .save_state_dict import save_state_dict, wait_async_save  # noqa: F401
