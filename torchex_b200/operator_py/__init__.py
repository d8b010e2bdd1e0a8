from .scatter_op import (GetPreSumFunction, ScatterData, ScatterMaxFunction, ScatterMeanFunction,
                         ScatterSumFunction, gather_back, getPreSum, ingroup_inds, ingroup_rank, scatter_max,
                         scatter_mean, scatter_mean_max, scatter_multi, scatter_sum, ScatterMeanMaxFunction)
from .timer import TorchTimer

__all__ = ["TorchTimer", "scatter_sum", "scatter_mean", "scatter_max", "getPreSum", "ScatterData",
           "ScatterSumFunction", "ScatterMeanFunction", "ScatterMaxFunction", "GetPreSumFunction",
           "ingroup_inds", "ingroup_rank", "gather_back", "scatter_mean_max", "scatter_multi", "ScatterMeanMaxFunction"]
