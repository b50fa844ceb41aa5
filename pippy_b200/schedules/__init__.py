from .actions import Action, Op, Schedule, add_send_recv, dump_csv, format_schedule, load_csv, validate
from .generators import (
    gpipe,
    interleaved_1f1b,
    looped_bfs,
    one_f_one_b,
    tuned_zero_bubble_placed,
    v_placement,
    with_reduce_grad,
    zero_bubble,
    zero_bubble_placed,
)
from .runtime import (
    PipelineSchedule,
    PipelineScheduleMulti,
    PipelineScheduleSingle,
    Schedule1F1B,
    ScheduleGPipe,
    ScheduleInterleaved1F1B,
    ScheduleInterleavedZeroBubble,
    ScheduleLoopedBFS,
    ScheduleTimeout,
    ScheduleZBVZeroBubble,
    ScheduleZeroBubble,
    sorted_batch_isend_irecv,
)
from .simulator import SimResult, ideal_bubble, simulate
from .trace import gather_measured_trace, measured_trace, simulated_trace, write_chrome_trace
