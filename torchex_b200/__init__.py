"""B200-native segmented scatter reduction with TorchEx's operator API.

Drop-in for the scatter part of ``torchex``: ``ScatterData``, ``scatter_sum``,
``scatter_mean``, ``scatter_max`` (and ``TorchTimer``), backed by hand-written
sm_100a kernels behind a C ABI (``include/texb_scatter.h``).
"""
from .operator_py import (ScatterData, TorchTimer, gather_back, getPreSum, ingroup_inds, ingroup_rank,
                          scatter_max, scatter_mean, scatter_mean_max, scatter_multi, scatter_sum)

__all__ = ["ScatterData", "TorchTimer", "getPreSum", "scatter_max", "scatter_mean", "scatter_sum",
           "ingroup_inds", "ingroup_rank", "gather_back", "scatter_mean_max", "scatter_multi"]
