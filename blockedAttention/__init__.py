"""Import-name alias of the upstream package: ``import blockedAttention`` gives
``blockGEMM`` and ``blockSoftmax`` (upstream blockedAttention/__init__.py:1-6),
served by blockedattention_b200."""
from blockedattention_b200.apply import blockAttention, blockAttentionTokenMajor, blockAttnScores, blockAttnScoresHost, blockAttnScoresTokenMajor, blockGEMM, blockSoftmax

__all__ = ["blockGEMM", "blockSoftmax", "blockAttention", "blockAttentionTokenMajor", "blockAttnScores", "blockAttnScoresHost", "blockAttnScoresTokenMajor"]
