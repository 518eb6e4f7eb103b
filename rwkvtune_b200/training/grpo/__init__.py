from ...engine.profiling import get_gpu_memory_info, monitor_memory_and_time
from .advantage import AdvantageCalculator
from .dataset import GRPODataBuffer, RepeatBatchSampler, create_grpo_dataloader
from .loss import BNPOLoss, DAPOLoss, DrGRPOLoss, GRPOLossBase, get_loss_function
from .utils import entropy_from_logits, selective_log_softmax

__all__ = ["AdvantageCalculator", "GRPODataBuffer", "RepeatBatchSampler", "create_grpo_dataloader", "GRPOLossBase",
           "DAPOLoss", "DrGRPOLoss", "BNPOLoss", "get_loss_function", "selective_log_softmax", "entropy_from_logits",
           "get_gpu_memory_info", "monitor_memory_and_time"]
