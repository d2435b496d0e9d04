"""Tensor-parallel partitioning of packed int4 weights (index arithmetic only).

Packed layout: `packed` [n][k/2] bytes and `scales` [n][k/group] (one row per output
channel, crates/yscv-kernels/src/ops/int4_matmul.rs:12-18), so

* column-parallel (split the output channels): rank r owns the contiguous row slice
  [r*n/G, (r+1)*n/G) of both arrays; no repacking, no collective when the consumer is
  sharded the same way (attention heads, SwiGLU);
* row-parallel (split K): rank r owns bytes [k0/2, k1/2) and scales [k0/g, k1/g) of
  every row, k0 = r*k/G; needs (k/G) % group == 0 so that no group straddles two ranks.
  Every rank produces an fp32 partial [m][n]; the partials are summed (all-reduce).

int8 QLinearMatMul / MatMulInteger (B [k][n] row-major, per-tensor or per-channel requant):
split the output channels; rank r owns the columns [r*n/G, (r+1)*n/G) of B and the matching
slice of every per-channel vector, A is replicated, the requant is per element, so the
ranks' byte outputs [m][n/G] are independent and are all-gathered.

Works on numpy arrays and torch tensors alike (plain slicing).
"""
from __future__ import annotations


def row_range(n: int, rank: int, world: int) -> tuple[int, int]:
    if n % world != 0:
        raise ValueError(f"{n} output channels do not split evenly across {world} ranks")
    per = n // world
    return rank * per, (rank + 1) * per


def col_range(k: int, group: int, rank: int, world: int) -> tuple[int, int]:
    if k % world != 0 or (k // world) % group != 0:
        raise ValueError(f"k={k} cannot be split across {world} ranks on group-{group} boundaries")
    per = k // world
    return rank * per, (rank + 1) * per


def shard_rows(packed, scales, rank: int, world: int):
    """Column-parallel shard: packed [n][k/2], scales [n][k/g] -> the rank's rows."""
    r0, r1 = row_range(packed.shape[0], rank, world)
    return packed[r0:r1], scales[r0:r1]


def shard_cols(packed, scales, group: int, rank: int, world: int):
    """Row-parallel shard: the rank's K slice of every row."""
    k = packed.shape[1] * 2
    k0, k1 = col_range(k, group, rank, world)
    return packed[:, k0 // 2:k1 // 2], scales[:, k0 // group:k1 // group]


def shard_activation_cols(act, group: int, rank: int, world: int):
    """The K slice of the activations [m][k] that goes with shard_cols."""
    k0, k1 = col_range(act.shape[-1], group, rank, world)
    return act[..., k0:k1]


def shard_i8_b_cols(b, rank: int, world: int):
    """N-shard of an int8 weight b [k][n]: the rank's output channels (a strided view)."""
    n0, n1 = row_range(b.shape[1], rank, world)
    return b[:, n0:n1]


def shard_channel_vector(v, rank: int, world: int):
    """The rank's slice of a per-output-channel vector (composite, correction, bias)."""
    n0, n1 = row_range(v.shape[0], rank, world)
    return v[n0:n1]


def assemble_cols(parts):
    """[G][m][n/G] gathered outputs -> [m][n] (torch tensors or numpy arrays)."""
    if hasattr(parts, "permute"):
        g, m, w = parts.shape
        return parts.permute(1, 0, 2).reshape(m, g * w)
    import numpy as np
    parts = np.asarray(parts)
    g, m, w = parts.shape
    return parts.transpose(1, 0, 2).reshape(m, g * w)


# ---- the exchange inside the tensor-parallel decode step ----------------------------------
# Host-side statement of the slot / tag arithmetic of csrc/decode_step.cu, so that it can be
# checked without a GPU. A step of `layers` layers has 2 * layers row-parallel GEMVs (output
# and down projection of every layer) followed by one greedy-token exchange. Every exchange
# writes {value, tag} words into slot (parity, source rank, row) of every peer's region.

def exchanges_per_step(layers: int) -> int:
    return 2 * layers + 1


def exchange_tag(step: int, layers: int, exchange: int) -> int:
    """32-bit tag of exchange number `exchange` (0 .. 2*layers) of decode step `step`; never 0,
    the value of a slot nobody has written yet."""
    tag = (step * exchanges_per_step(layers) + exchange + 1) & 0xFFFFFFFF
    return tag


def exchange_parity(step: int, layers: int, exchange: int) -> int:
    """Which of the two slot sets an exchange uses: the GEMV exchanges alternate (there is an
    even number of them per step, so the alternation continues across steps); the token
    exchange has slots of its own and alternates by step."""
    return (exchange & 1) if exchange < 2 * layers else (step & 1)


def exchange_slot(parity: int, src_rank: int, row: int, world: int, rows_cap: int) -> int:
    """Word index of (parity, source rank, row) in a rank's exchange region."""
    return (parity * world + src_rank) * rows_cap + row


def sum_in_rank_order(partials):
    """What every rank computes from the world's partial sums: p0 + p1 + ... in rank order,
    hence bit-identical on every rank."""
    total = partials[0].copy()
    for p in partials[1:]:
        total = total + p
    return total
