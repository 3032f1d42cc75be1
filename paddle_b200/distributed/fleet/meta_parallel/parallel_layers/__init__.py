from .pp_layers import LayerDesc, PipelineLayer, PipelineLayerChunk, SegmentLayers, SharedLayerDesc  # noqa: F401
