"""
Who owns what in the sharded optimizer — pure Python, no tensors, testable anywhere.

The ownership rules are those of the reference's ZeRO-2-style optimizer so that
per-rank optimizer checkpoints stay interchangeable (reference: nanochat/optim.py):
  * AdamW parameters with fewer than 1024 elements are replicated: every rank
    averages the full gradient and keeps full state (optim.py:282-285).
  * Larger AdamW parameters are cut along dim 0 into `world` equal row slices;
    rank r owns rows [r*rows/world, (r+1)*rows/world) (optim.py:286-292,333-335).
  * A Muon group of K same-shape matrices is split into chunks of ceil(K/world)
    consecutive matrices; rank r owns matrices [r*chunk, min(K, (r+1)*chunk))
    and keeps state buffers with `chunk` rows even if it owns fewer
    (optim.py:302,373-382).
"""

from dataclasses import dataclass

SMALL_PARAM_NUMEL = 1024


@dataclass(frozen=True)
class AdamWShard:
    replicated: bool
    row_start: int
    row_end: int

    @property
    def rows(self):
        return self.row_end - self.row_start


@dataclass(frozen=True)
class MuonShard:
    chunk: int        # matrices per rank (state buffer leading dim)
    start: int        # first owned matrix index
    num_owned: int    # how many this rank really owns (may be < chunk, even 0)
    padded: int       # chunk * world, the padded stack length a collective would need


def adamw_shard(shape, rank: int, world: int) -> AdamWShard:
    numel = 1
    for s in shape:
        numel *= s
    rows = shape[0] if len(shape) > 0 else 1
    if world == 1 or numel < SMALL_PARAM_NUMEL:
        return AdamWShard(True, 0, rows)
    if rows % world != 0:
        raise ValueError(f"AdamW sharding needs shape[0] ({rows}) divisible by world size ({world})")
    per = rows // world
    return AdamWShard(False, rank * per, (rank + 1) * per)


def muon_shard(num_params: int, rank: int, world: int) -> MuonShard:
    chunk = -(-num_params // world)
    start = rank * chunk
    owned = min(chunk, max(0, num_params - start))
    return MuonShard(chunk, start, owned, chunk * world)


def muon_owner(index: int, num_params: int, world: int) -> int:
    """Rank that owns matrix `index` of a K-matrix Muon group."""
    return index // (-(-num_params // world))
