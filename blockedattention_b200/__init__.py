"""blockedattention_b200: varlen blocked GEMM + varlen row softmax for NVIDIA B200.

Drop-in for the two operators of Sophie10001b/blockedAttention
(``blockGEMM``, ``blockSoftmax``) over the same packed head-major layout, on
hand-written sm_100a kernels behind a C ABI (``include/blkattn.h``).
"""
from .apply import blockAttention, blockAttentionTokenMajor, blockAttnScores, blockAttnScoresHost, blockAttnScoresTokenMajor, blockGEMM, blockSoftmax, check_plans, clear_plan_cache
from .plan import GemmPlan, SoftmaxPlan

__all__ = ["blockGEMM", "blockSoftmax", "blockAttention", "blockAttentionTokenMajor", "blockAttnScores", "blockAttnScoresHost", "blockAttnScoresTokenMajor", "GemmPlan", "SoftmaxPlan", "clear_plan_cache", "check_plans"]
