from .bootstrap import DistContext, init_distributed, shutdown
from .flat import FlatParamSpace, ParamGroupSpec, build_param_groups
from .zero import ZeroOptimizer, merge_shards

__all__ = ["DistContext", "init_distributed", "shutdown", "FlatParamSpace", "ParamGroupSpec", "build_param_groups",
           "ZeroOptimizer", "merge_shards"]
