"""B200-native MoBA (Mixture of Block Attention) causal prefill.

Drop-in for the package the reference loads by path
(backends/_mthreads/ops/moba/__init__.py:2-3 exports ``parallel_moba``)."""
from .parallel import moba_attn_varlen, moba_forward, parallel_moba

__all__ = ["parallel_moba", "moba_attn_varlen", "moba_forward"]
