from .scatter_op import (GetPreSumFunction, ScatterData, ScatterMaxFunction, ScatterMeanFunction,
                         ScatterSumFunction, getPreSum, scatter_max, scatter_mean, scatter_sum)
from .timer import TorchTimer

__all__ = ["TorchTimer", "scatter_sum", "scatter_mean", "scatter_max", "getPreSum", "ScatterData",
           "ScatterSumFunction", "ScatterMeanFunction", "ScatterMaxFunction", "GetPreSumFunction"]
