from .crash_dump import describe_step_failure, dump_step_failure, tensor_summary
from .logging import get_logger
from .stages import enable_stages, profile_to, stage, stages_enabled
