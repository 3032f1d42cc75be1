"""``paddle.device.cuda.streams`` (python/paddle/device/cuda/streams.py)."""
import torch

Stream = torch.cuda.Stream
Event = torch.cuda.Event
