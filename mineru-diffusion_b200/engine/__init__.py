from .config import Config, DecoderConfig
from .sampling_params import SamplingParams
from .sequence import Sequence, SequenceStatus
from .block_manager import BlockManager
from .scheduler import Scheduler
from .context import Context

__all__ = ["Config", "DecoderConfig", "SamplingParams", "Sequence", "SequenceStatus", "BlockManager",
           "Scheduler", "Context"]
