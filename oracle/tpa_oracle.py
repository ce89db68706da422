"""CPU oracle for the Tensor Product Attention forward and its ring wrapper.

TEST INFRASTRUCTURE ONLY.  This file is a CPU restatement (numpy, plus a torch
variant for speed) of the arithmetic the reference writes out in

    tpa/tpa_test.py:22-57    reference(): rank-mean materialisation, segment / causal bias
    tpa/mha.py:23-37         _mha_fwd(): softmax(sm_scale * Q K^T + bias) V
    tpa/tpa.py:220-242       _lse, _lse_accum
    tpa/tpa.py:290-443       _fwd_kernel: block-wise online (LSE-normalised) softmax
    tpa/ring_tpa.py:60-112   _ring_tpa_fwd: N-step (o, lse) merge + rotation of K/V factors

Only tests, the smoke check and the benchmark's CPU-baseline leg may import it;
the shipped library never does.

Parity pin: the reference is pure Python on JAX + Pallas and JAX is not
installed where this was built, so the restatement is pinned against outputs
obtained by executing the reference's own, unmodified source files on top of a
numpy stand-in for the small slice of the jax API they touch
(tests/golden/make_golden.py, tests/golden/_jax_standin.py).  What this does
not pin is XLA's own floating-point evaluation order; the fixtures are compared
at the reference's own test tolerance (rtol = atol = 1e-3) and, because both
sides are numpy fp32/fp64, in practice agree to ~1e-6.
"""

from __future__ import annotations

import math

import numpy as np

__all__ = [
    "split_factors",
    "materialize",
    "lse",
    "lse_accum",
    "tpa_reference",
    "tpa_fwd_blockwise",
    "ring_tpa_reference",
    "make_factors",
    "segment_ids",
    "position_mask",
    "key_positions",
    "rope_tables",
    "apply_rope",
    "attn_flops",
]


# --------------------------------------------------------------------------- inputs


def make_factors(seed, b, lq, lk, rq, rk, h, dk, dv, dist="normal", dtype=np.float32):
    """Seeded synthetic factors in the reference's concatenated layout.

    Returns q[b,lq,rq,h+dk], k[b,lk,rk,h+dk], v[b,lk,rk,h+dv] with the head
    factor A in [..., :h] and the dim factor B in [..., h:] (tpa/tpa.py:477-479).

    dist="normal": A ~ N(0,1), B ~ N(0,1)/sqrt(d) (the benchmark configurations).
    dist="uniform": U[0,1) everywhere (tpa/tpa_test.py:86-91).
    The stream is numpy Philox keyed by `seed`; draw order A_Q,B_Q,A_K,B_K,A_V,B_V.
    """
    rng = np.random.Generator(np.random.Philox(key=seed))

    def draw(shape, scale):
        if dist == "normal":
            return rng.standard_normal(shape, dtype=np.float32) * np.float32(scale)
        if dist == "uniform":
            return rng.random(shape, dtype=np.float32)
        raise ValueError(dist)

    qa = draw((b, lq, rq, h), 1.0)
    qb = draw((b, lq, rq, dk), dk**-0.5)
    ka = draw((b, lk, rk, h), 1.0)
    kb = draw((b, lk, rk, dk), dk**-0.5)
    va = draw((b, lk, rk, h), 1.0)
    vb = draw((b, lk, rk, dv), dv**-0.5)
    q = np.concatenate([qa, qb], axis=-1).astype(dtype)
    k = np.concatenate([ka, kb], axis=-1).astype(dtype)
    v = np.concatenate([va, vb], axis=-1).astype(dtype)
    return q, k, v


def segment_ids(b, length, segment_size):
    """arange(l) // segment_size repeated over batch (tpa/tpa_test.py:93-99)."""
    ids = (np.arange(length) // segment_size).astype(np.int32)
    return np.broadcast_to(ids, (b, length)).copy()


def attn_flops(b, h, d, lq, lk, causal):
    """Algorithmic FLOPs of the two dense contractions (QK^T and PV), 2 FLOP per MAC."""
    pairs = lq * (lq + 1) // 2 if (causal and lq == lk) else lq * lk
    return 4.0 * b * h * d * pairs


# --------------------------------------------------------------------------- pieces


def split_factors(x, num_heads):
    """tpa/tpa.py:477-479 — head factor A = x[..., :h], dim factor B = x[..., h:]."""
    return x[..., :num_heads], x[..., num_heads:]


def materialize(q, k, v, num_heads, dtype=np.float64):
    """tpa/tpa_test.py:36-44 — Q, K, V as rank means of outer products."""
    qa, qb = split_factors(np.asarray(q, dtype=dtype), num_heads)
    ka, kb = split_factors(np.asarray(k, dtype=dtype), num_heads)
    va, vb = split_factors(np.asarray(v, dtype=dtype), num_heads)
    rq = qa.shape[2]
    rk = ka.shape[2]
    q_ = np.einsum("blrh,blrd->blhd", qa, qb) / rq
    k_ = np.einsum("blrh,blrd->blhd", ka, kb) / rk
    v_ = np.einsum("blrh,blrd->blhd", va, vb) / rk
    return q_, k_, v_


def lse(x):
    """tpa/tpa.py:220-225 — logsumexp over the last axis, -inf for empty rows."""
    with np.errstate(invalid="ignore", divide="ignore"):
        m = np.max(x, axis=-1)
        out = m + np.log(np.sum(np.exp(x - m[..., None]), axis=-1))
    return np.where(np.isneginf(m), -np.inf, out)


def lse_accum(a, b):
    """tpa/tpa.py:228-242 — pairwise merge max + log(1 + exp(min - max))."""
    with np.errstate(invalid="ignore", divide="ignore"):
        hi = np.maximum(a, b)
        lo = np.minimum(a, b)
        out = hi + np.log(1 + np.exp(lo - hi))
    return np.where(np.isneginf(hi), -np.inf, out)


def position_mask(q_pos, k_pos, causal, window=0, dilation=1):
    """Keep-mask [lq, lk] from positions: the causal rule of tpa/tpa_test.py:52-54 /
    tpa/tpa.py:376-379 (query position >= key position), and the sliding-window / dilated
    variants the reference only plans (tpa/ring_tpa.py:5-7, tpa/tpa.py:31-32), defined here as:
    with diff = q_pos - k_pos a pair is kept iff |diff| < window * dilation and
    diff % dilation == 0 (and diff >= 0 when causal), i.e. `window` keys at stride `dilation`
    behind the query, and as many ahead when not causal.  window = 0: no window."""
    diff = np.asarray(q_pos)[:, None] - np.asarray(k_pos)[None, :]
    keep = np.ones(diff.shape, dtype=bool)
    if causal:
        keep &= diff >= 0
    dilation = max(1, int(dilation))
    if window and window > 0:
        span = int(window) * dilation
        keep &= (diff < span) & (-diff < span)
    if dilation > 1:
        keep &= diff % dilation == 0
    return keep


def key_positions(lk, k_offset=0, kv_parts=1, per_part=False):
    """Position of every key in the mask comparisons.  With `per_part` the keys are `kv_parts`
    equal parts (the visiting shards of a ring) and each is compared on its index inside its own
    part, which is what the reference's ring does at every step (tpa/ring_tpa.py:73-79)."""
    idx = np.arange(lk)
    if per_part and kv_parts > 1:
        idx = idx % (lk // kv_parts)
    return idx + k_offset


def _mask(b, lq, lk, q_seg, kv_seg, causal, q_offset=0, k_offset=0, window=0, dilation=1, kv_parts=1,
          per_part=False):
    """Boolean keep-mask [b, lq, lk] (tpa/tpa_test.py:46-55; tpa/tpa.py:369-383)."""
    keep = np.ones((b, lq, lk), dtype=bool)
    if q_seg is not None:
        assert kv_seg is not None
        keep &= np.asarray(q_seg)[:, :, None] == np.asarray(kv_seg)[:, None, :]
    if causal or window or dilation > 1:
        keep &= position_mask(np.arange(lq) + q_offset, key_positions(lk, k_offset, kv_parts, per_part),
                              causal, window, dilation)[None]
    return keep


# --------------------------------------------------------------------------- rotary embedding


def rope_tables(length, d, base=10000.0, dtype=np.float32):
    """cos / sin tables [length, d / 2] of the rotary position embedding (Su et al., RoFormer):
    angle of position t, pair c = t * base ** (-2 c / d)."""
    inv = base ** (-np.arange(0, d, 2, dtype=np.float64) / d)
    ang = np.arange(length, dtype=np.float64)[:, None] * inv[None, :]
    return np.cos(ang).astype(dtype), np.sin(ang).astype(dtype)


def apply_rope(x, num_heads, cos, sin, offset=0):
    """Rotate the dim factor B = x[..., h:] of a concatenated factor array [b, l, r, h + d].

    The reference has no rotary embedding (its README links the paper only); Tensor Product
    Attention applies it to the B factors of q and k before the rank sum, which equals rotating
    the rebuilt Q and K rows because the rotation is linear and the same for every rank:
    columns (2c, 2c + 1) of row t turn by the angle of table row t + offset,
    (x, y) -> (x cos - y sin, x sin + y cos).  Returns a new array; A is untouched."""
    x = np.array(x, dtype=np.float64 if np.asarray(x).dtype == np.float64 else np.float32, copy=True)
    l = x.shape[1]
    c = np.asarray(cos)[offset:offset + l][None, :, None, :].astype(x.dtype)
    s_ = np.asarray(sin)[offset:offset + l][None, :, None, :].astype(x.dtype)
    b = x[..., num_heads:]
    ev, od = b[..., 0::2].copy(), b[..., 1::2].copy()
    b[..., 0::2] = ev * c - od * s_
    b[..., 1::2] = ev * s_ + od * c
    return x


# --------------------------------------------------------------------------- (i) materialised definition


def tpa_reference(
    q,
    k,
    v,
    num_heads,
    q_segment_ids=None,
    kv_segment_ids=None,
    sm_scale=1.0,
    causal=False,
    dtype=np.float64,
    q_offset=0,
    k_offset=0,
    return_lse=False,
    window=0,
    dilation=1,
    kv_parts=1,
    per_part=False,
):
    """Definition of the result: tpa/tpa_test.py:22-57 + tpa/mha.py:23-37.

    Rows whose every key is masked come out NaN (softmax of all -inf), which is
    also what the kernel writes (tpa/tpa.py:439).  `q_offset/k_offset` shift the
    causal comparison to global positions; the reference has no such argument
    (both are 0 there).  `window`, `dilation`, `kv_parts`, `per_part`: see position_mask and
    key_positions.
    """
    q_, k_, v_ = materialize(q, k, v, num_heads, dtype)
    b, lq = q_.shape[:2]
    lk = k_.shape[1]
    x = np.einsum("bqhd,bkhd->bhqk", q_, k_) * dtype(sm_scale)
    keep = _mask(b, lq, lk, q_segment_ids, kv_segment_ids, causal, q_offset, k_offset, window, dilation, kv_parts,
                 per_part)
    x = np.where(keep[:, None], x, -np.inf)
    with np.errstate(invalid="ignore", divide="ignore"):
        m = np.max(x, axis=-1, keepdims=True)
        e = np.exp(x - m)
        p = e / np.sum(e, axis=-1, keepdims=True)  # NaN for empty rows, as jax.nn.softmax
    o = np.einsum("bhqk,bkhd->bqhd", p, v_)
    if return_lse:
        return o, np.transpose(lse(x), (0, 2, 1))  # [b, lq, h]
    return o


def tpa_bwd_reference(
    q,
    k,
    v,
    do,
    num_heads,
    q_segment_ids=None,
    kv_segment_ids=None,
    sm_scale=1.0,
    causal=False,
    dtype=np.float64,
    q_offset=0,
    k_offset=0,
):
    """Gradients of `tpa_reference` with respect to the concatenated factors, given `do`.

    Follows the materialising branch of the backward kernel (tpa/tpa.py:777-799):
    p = exp(x - lse) with NaN -> 0 (tpa/tpa.py:676-677), delta = nansum(o * do)
    (tpa/tpa.py:976-980), ds = p (do v^T - delta) sm_scale, dq = ds k, dk = ds^T q,
    dv = p^T do, and the factor contraction da = dX b / R, db = dX a / R
    (tpa/tpa.py:779-781, 789-791, 796-799).  A query row that sees no key has p = 0 and a
    NaN-free delta, so it contributes nothing, here as there.  Two deliberate differences,
    both outside what the reference's own tests execute (tpa/tpa_test.py:128-205 is
    non-causal with at most two heads):
      * db sums over ALL heads.  The reference's program for head block i overwrites the
        db block written by head block i-1 (tpa/tpa.py:929,933 ignore the head index),
        which is only right while num_heads <= block_h.
      * the causal trip count of the reference (tpa/tpa.py:811-812) is not followed; the
        mask itself defines which pairs contribute.
    Pinned by tests/golden/bwd_matrix.npz: the reference's own _tpa_bwd executed on the
    24 shapes of its backward test.
    Returns (dq, dk, dv) shaped like q, k, v.
    """
    return tpa_bwd_block(q, k, v, do, None, None, num_heads, q_segment_ids, kv_segment_ids, sm_scale,
                         causal, dtype, q_offset, k_offset)


def tpa_bwd_block(
    q,
    k,
    v,
    do,
    o,
    l,
    num_heads,
    q_segment_ids=None,
    kv_segment_ids=None,
    sm_scale=1.0,
    causal=False,
    dtype=np.float64,
    q_offset=0,
    k_offset=0,
):
    """One block of the backward for given residuals `o` [b,lq,h,dv] and `l` [b,lq,h] (the
    operands of _bwd, tpa/tpa.py:823-839): what a ring step computes with the LSE of the whole
    ring (tpa/ring_tpa.py:147-156).  `o = l = None`: residuals of this block's own forward."""
    qa, qb = split_factors(np.asarray(q, dtype), num_heads)
    ka, kb = split_factors(np.asarray(k, dtype), num_heads)
    va, vb = split_factors(np.asarray(v, dtype), num_heads)
    do = np.asarray(do, dtype)
    rq, rk = qa.shape[2], ka.shape[2]
    q_, k_, v_ = materialize(q, k, v, num_heads, dtype)
    b, lq = q_.shape[:2]
    lk = k_.shape[1]
    x = np.einsum("bqhd,bkhd->bhqk", q_, k_) * dtype(sm_scale)
    keep = _mask(b, lq, lk, q_segment_ids, kv_segment_ids, causal, q_offset, k_offset)
    x = np.where(keep[:, None], x, -np.inf)
    with np.errstate(invalid="ignore", divide="ignore"):
        lcol = lse(x)[..., None] if l is None else np.transpose(np.asarray(l, dtype), (0, 2, 1))[..., None]
        p = np.exp(x - lcol)  # [b, h, lq, lk]
    p = np.where(np.isnan(p), 0.0, p)
    if o is None:
        o = np.einsum("bhqk,bkhd->bqhd", p, v_)
    delta = np.nansum(np.asarray(o, dtype) * do, axis=-1).transpose(0, 2, 1)[..., None]  # tpa/tpa.py:979
    dp = np.einsum("bqhd,bkhd->bhqk", do, v_) - delta
    ds = p * dp * dtype(sm_scale)
    dq_ = np.einsum("bhqk,bkhd->bqhd", ds, k_)
    dk_ = np.einsum("bhqk,bqhd->bkhd", ds, q_)
    dv_ = np.einsum("bhqk,bqhd->bkhd", p, do)

    def contract(dx, a, bf, rank):
        da = np.einsum("blhd,blrd->blrh", dx, bf) / rank
        db = np.einsum("blhd,blrh->blrd", dx, a) / rank
        return np.concatenate([da, db], axis=-1)

    return contract(dq_, qa, qb, rq), contract(dk_, ka, kb, rk), contract(dv_, va, vb, rk)


# --------------------------------------------------------------------------- (ii) block-wise kernel semantics


def tpa_fwd_blockwise(
    q,
    k,
    v,
    num_heads,
    q_segment_ids=None,
    kv_segment_ids=None,
    sm_scale=1.0,
    causal=False,
    block_q=128,
    block_kv=128,
    dtype=np.float64,
):
    """Restatement of _fwd / _fwd_kernel (tpa/tpa.py:473-543, 290-443).

    Per batch element and query block: loop over key/value blocks, rebuild K
    and V for the block, masked logits, l = lse_accum(l_prev, lse(x)),
    p = exp(x - l), o = exp(l_prev - l) * o + p V (o stays normalised every
    step), causal trip count ceil(block_q (q_i + 1) / block_kv), NaN rows where
    l stays -inf.  Returns (o[b,lq,h,dv], lse[b,lq,h]).
    """
    q_, k_, v_ = materialize(q, k, v, num_heads, dtype)
    b, lq, h, _ = q_.shape
    lk = k_.shape[1]
    dv = v_.shape[-1]
    block_q = min(block_q, lq)  # tpa/tpa.py:485-486
    block_kv = min(block_kv, lk)
    assert lq % block_q == 0, (lq, block_q)  # tpa/tpa.py:489-490
    assert lk % block_kv == 0, (lk, block_kv)
    o_out = np.empty((b, lq, h, dv), dtype=dtype)
    l_out = np.empty((b, lq, h), dtype=dtype)
    for bi in range(b):
        for qi in range(lq // block_q):
            qs = slice(qi * block_q, (qi + 1) * block_q)
            qq = q_[bi, qs]  # [bq, h, dk]
            o = np.zeros((h, block_q, dv), dtype=dtype)
            l = np.full((h, block_q), -np.inf, dtype=dtype)
            if causal:
                nkv = (block_q * (qi + 1) + block_kv - 1) // block_kv  # tpa/tpa.py:428
                nkv = min(nkv, -(-lk // block_kv))
            else:
                nkv = -(-lk // block_kv)
            for ki in range(nkv):
                ks = slice(ki * block_kv, (ki + 1) * block_kv)
                x = np.einsum("qhd,khd->hqk", qq, k_[bi, ks]) * dtype(sm_scale)
                keep = np.ones((block_q, block_kv), dtype=bool)
                if kv_segment_ids is not None:
                    keep &= (
                        np.asarray(q_segment_ids)[bi, qs][:, None]
                        == np.asarray(kv_segment_ids)[bi, ks][None, :]
                    )
                if causal:
                    span_q = qi * block_q + np.arange(block_q)
                    span_k = ki * block_kv + np.arange(block_kv)
                    keep &= span_q[:, None] >= span_k[None, :]
                x = np.where(keep[None], x, -np.inf)
                l_new = lse_accum(l, lse(x))
                with np.errstate(invalid="ignore"):
                    p = np.exp(x - l_new[..., None])
                    p = np.where(np.isneginf(l_new[..., None]), 0.0, p)
                    corr = np.exp(l - l_new)
                    corr = np.where(np.isneginf(l_new), 0.0, corr)
                o = corr[..., None] * o + np.einsum("hqk,khd->hqd", p, v_[bi, ks])
                l = l_new
            o = np.where(np.isneginf(l)[..., None], np.nan, o)
            o_out[bi, qs] = np.transpose(o, (1, 0, 2))
            l_out[bi, qs] = np.transpose(l, (1, 0))
    return o_out, l_out


# --------------------------------------------------------------------------- (iii) ring


def ring_tpa_reference(
    q,
    k,
    v,
    q_segment_ids,
    kv_segment_ids,
    num_heads,
    n_shards,
    sm_scale=1.0,
    causal=False,
    mask_mode="reference_local",
    dtype=np.float64,
):
    """Restatement of _ring_tpa_fwd over `n_shards` simulated ranks (tpa/ring_tpa.py:60-112).

    The global arrays are cut into contiguous length shards (the PartitionSpec of
    tpa/ring_tpa_test.py:108,125-132).  Rank r keeps its query shard; at step s it
    sees the K/V shard that started on rank (r - s) mod N, because every step
    rotates i -> i+1 (tpa/ring_tpa.py:34-38,96).  Partials merge with
    lse_accum and exp(l - l_next) weights with NaN -> 0 (tpa/ring_tpa.py:82-91);
    rows that never saw a key are NaN at the end (tpa/ring_tpa.py:109).

    mask_mode="reference_local": the causal mask is applied on local indices at
    every step, exactly as the reference does (no shard offset reaches the block
    kernel, tpa/ring_tpa.py:73-79, tpa/tpa.py:376-379).
    mask_mode="global": causal on global positions (equals tpa(causal=True) on the
    unsharded input); not what the reference computes.
    """
    b, lq = q.shape[:2]
    lk = k.shape[1]
    assert lq % n_shards == 0 and lk % n_shards == 0
    sq, sk = lq // n_shards, lk // n_shards
    dv = v.shape[-1] - num_heads
    out = np.empty((b, lq, num_heads, dv), dtype=dtype)
    for r in range(n_shards):
        qs = slice(r * sq, (r + 1) * sq)
        o = np.zeros((b, sq, num_heads, dv), dtype=dtype)
        l = np.full((b, sq, num_heads), -np.inf, dtype=dtype)
        for step in range(n_shards):
            src = (r - step) % n_shards
            ks = slice(src * sk, (src + 1) * sk)
            q_off, k_off = (r * sq, src * sk) if mask_mode == "global" else (0, 0)
            o_, l_ = tpa_reference(
                q[:, qs],
                k[:, ks],
                v[:, ks],
                num_heads,
                None if q_segment_ids is None else q_segment_ids[:, qs],
                None if kv_segment_ids is None else kv_segment_ids[:, ks],
                sm_scale=sm_scale,
                causal=causal,
                dtype=dtype,
                q_offset=q_off,
                k_offset=k_off,
                return_lse=True,
            )
            l_next = lse_accum(l, l_)
            with np.errstate(invalid="ignore"):
                o = np.nan_to_num(o * np.exp(l - l_next)[..., None], nan=0.0)
                o_ = np.nan_to_num(o_ * np.exp(l_ - l_next)[..., None], nan=0.0)
            o = o + o_
            l = l_next
        out[:, qs] = np.where(np.isneginf(l)[..., None], np.nan, o)
    return out


def ring_tpa_bwd_reference(
    q,
    k,
    v,
    q_segment_ids,
    kv_segment_ids,
    do,
    num_heads,
    n_shards,
    sm_scale=1.0,
    causal=False,
    mask_mode="reference_local",
    dtype=np.float64,
):
    """Restatement of _ring_tpa_bwd over `n_shards` simulated ranks (tpa/ring_tpa.py:115-172):
    every (query shard r, key shard src) block runs the block backward with the o and LSE of the
    whole ring forward; dq sums on r, dk / dv travel with the K/V shard and sum on src."""
    b, lq = q.shape[:2]
    lk = k.shape[1]
    sq, sk = lq // n_shards, lk // n_shards
    o = ring_tpa_reference(q, k, v, q_segment_ids, kv_segment_ids, num_heads, n_shards, sm_scale, causal,
                           mask_mode, dtype)
    # LSE of the whole ring: lse_accum over the steps (tpa/ring_tpa.py:82)
    l = np.full((b, lq, num_heads), -np.inf, dtype=dtype)
    blocks = []
    for r in range(n_shards):
        for src in range(n_shards):
            qs, ks = slice(r * sq, (r + 1) * sq), slice(src * sk, (src + 1) * sk)
            offs = (r * sq, src * sk) if mask_mode == "global" else (0, 0)
            blocks.append((qs, ks, offs))
            _, l_ = tpa_reference(q[:, qs], k[:, ks], v[:, ks], num_heads,
                                  None if q_segment_ids is None else q_segment_ids[:, qs],
                                  None if kv_segment_ids is None else kv_segment_ids[:, ks],
                                  sm_scale, causal, dtype, offs[0], offs[1], return_lse=True)
            l[:, qs] = lse_accum(l[:, qs], l_)
    dq, dk, dv = (np.zeros(x.shape, dtype=dtype) for x in (q, k, v))
    for qs, ks, offs in blocks:
        g = tpa_bwd_block(q[:, qs], k[:, ks], v[:, ks], do[:, qs], o[:, qs], l[:, qs], num_heads,
                          None if q_segment_ids is None else q_segment_ids[:, qs],
                          None if kv_segment_ids is None else kv_segment_ids[:, ks],
                          sm_scale, causal, dtype, offs[0], offs[1])
        dq[:, qs] += g[0]
        dk[:, ks] += g[1]
        dv[:, ks] += g[2]
    return dq, dk, dv


# --------------------------------------------------------------------------- torch variant (large cases, CPU baseline)


def tpa_reference_torch(
    q,
    k,
    v,
    num_heads,
    q_segment_ids=None,
    kv_segment_ids=None,
    sm_scale=1.0,
    causal=False,
    rows=None,
    q_offset=0,
    k_offset=0,
    dtype=None,
    return_lse=False,
    window=0,
    dilation=1,
    kv_parts=1,
    per_part=False,
):
    """Same definition as tpa_reference, in torch on the host cores (all threads).

    `rows` (1-D index tensor) restricts the computation to those query rows so
    that very long sequences can be spot-checked; the result then has
    len(rows) in place of lq.  Materialise + dense softmax, one head at a time
    to bound memory.
    """
    import torch

    dtype = dtype or torch.float32
    q = torch.as_tensor(q).to(dtype)
    k = torch.as_tensor(k).to(dtype)
    v = torch.as_tensor(v).to(dtype)
    h = num_heads
    b, lq, rq, _ = q.shape
    lk, rk = k.shape[1], k.shape[2]
    dv = v.shape[-1] - h
    q_pos = torch.arange(lq)
    if rows is not None:
        rows = torch.as_tensor(rows, dtype=torch.long)
        q = q[:, rows]
        q_pos = rows
    nq = q.shape[1]
    keep = None
    if q_segment_ids is not None:
        qs = torch.as_tensor(q_segment_ids)
        if rows is not None:
            qs = qs[:, rows]
        keep = qs[:, :, None] == torch.as_tensor(kv_segment_ids)[:, None, :]
    if causal or window or dilation > 1:
        c = torch.from_numpy(position_mask(q_pos.numpy() + q_offset, key_positions(lk, k_offset, kv_parts, per_part),
                                           causal, window, dilation))
        keep = c[None] if keep is None else keep & c[None]
    o = torch.empty((b, nq, h, dv), dtype=dtype)
    l = torch.empty((b, nq, h), dtype=dtype)
    for hi in range(h):
        # rank mean as a broadcast multiply + sum: torch threads it, an einsum with these shapes
        # becomes l tiny matrix products on one core
        qh = (q[..., hi, None] * q[..., h:]).sum(2) / rq
        kh = (k[..., hi, None] * k[..., h:]).sum(2) / rk
        vh = (v[..., hi, None] * v[..., h:]).sum(2) / rk
        x = torch.einsum("bqd,bkd->bqk", qh, kh) * sm_scale
        if keep is not None:
            x = x.masked_fill(~keep, -math.inf)
        if return_lse:
            l[:, :, hi] = torch.logsumexp(x, dim=-1)
        p = torch.softmax(x, dim=-1)  # NaN for empty rows
        o[:, :, hi] = torch.einsum("bqk,bkd->bqd", p, vh)
    if return_lse:
        return o, l
    return o
