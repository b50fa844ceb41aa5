"""pippy_b200: pipeline parallelism for PyTorch on Blackwell (sm_100a)."""
from ._debug import logger  # noqa: F401
from .backward import stage_backward, stage_backward_input, stage_backward_weight  # noqa: F401
from .checkpoint import load_checkpoint, save_checkpoint  # noqa: F401
from .ir import (  # noqa: F401
    ArgsChunkSpec,
    KwargsChunkSpec,
    LossWrapper,
    MultiUseParameterConfig,
    Pipe,
    PipeSequential,
    PipeSplitWrapper,
    SplitPoint,
    TrivialLossWrapper,
    annotate_split_points,
    pipe_split,
    pipeline,
)
from .manual_stage import ManualPipelineStage, get_stage_shapes, validate_stage_shapes  # noqa: F401
from .microbatch import (  # noqa: F401
    TensorChunkSpec,
    merge_chunks,
    split_args_kwargs_into_chunks,
    sum_reducer,
)
from .pipeline_stage import PipelineStage  # noqa: F401
from .split_policies import split_by_graph, split_into_equal_size, split_on_size_threshold  # noqa: F401
from .schedules import (  # noqa: F401
    Schedule1F1B,
    ScheduleGPipe,
    ScheduleInterleaved1F1B,
    ScheduleInterleavedZeroBubble,
    ScheduleLoopedBFS,
    ScheduleZBVZeroBubble,
    ScheduleZeroBubble,
)

__version__ = "0.1.0"
