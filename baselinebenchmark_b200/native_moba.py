"""Counterpart of backends/_mthreads/ops/moba/native_moba.py for harness code
that asks the package whether its native sparse path is eligible
(benchmarks/moba_compare.py:130, :203 call ``native_moba._supported(q)``)."""
import torch


def _supported(q: torch.Tensor) -> bool:
    """True where the tcgen05 dense stage runs: CUDA bf16 or fp16, head_dim 64 or 128, sm_100
    (the reference's native path has the same head dims, native_moba.py:30; 96 and 256 run
    the mma.sync dense stage, the counterpart of the reference's generic path)."""
    if q.device.type != "cuda" or q.dtype not in (torch.bfloat16, torch.float16) or q.shape[-1] not in (64, 128):
        return False
    return torch.cuda.get_device_capability(q.device)[0] == 10
