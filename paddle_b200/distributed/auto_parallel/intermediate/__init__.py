from .parallelize import (ColWiseParallel, LocalLayer, PrepareLayerInput, PrepareLayerOutput, RowWiseParallel,  # noqa: F401
                          SequenceParallelBegin, SequenceParallelDisable, SequenceParallelEnable,
                          SequenceParallelEnd, SplitPoint, parallelize, to_distributed)
