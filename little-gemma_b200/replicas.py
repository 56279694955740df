"""Replica-per-GPU aggregation: batch-1 decode does not shard, so N GPUs serve N independent
sessions with no collective on the data path.  Whole-job throughput is the tokens all replicas
emitted divided by the slowest replica's device time."""
from __future__ import annotations

from typing import Dict, List, Sequence


def aggregate(rows: Sequence[Sequence[float]]) -> Dict[str, float]:
    """rows[r] = [tokens emitted, device ms, e2e tokens, e2e seconds, stream identical (0/1)] of rank r."""
    if not rows:
        raise ValueError("no replica results")
    tokens = sum(r[0] for r in rows)
    max_ms = max(r[1] for r in rows)
    e2e_tokens = sum(r[2] for r in rows)
    e2e_s = max(r[3] for r in rows)
    return {
        "tok_s": tokens / (max_ms * 1e-3) if max_ms > 0 else 0.0,
        "max_ms": max_ms,
        "e2e_tok_s": e2e_tokens / e2e_s if e2e_s > 0 else 0.0,
        "identical": float(all(r[4] >= 0.5 for r in rows)),
        "n": float(len(rows)),
    }


def session_seed(rank: int) -> int:
    """Prompt seed of replica `rank` (each replica runs its own session)."""
    return 100 + rank
