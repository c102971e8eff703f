"""CPU oracle for xDiT's Unified-Sequence-Parallel (USP) attention path.  TEST INFRASTRUCTURE ONLY.

This module is a plain numpy restatement of the reference algorithm; it is the *checker*
that tests, the smoke entry and the benchmark's CPU-baseline leg compare the CUDA path with.
Nothing in the shipped package may import it.

Parity status: **pinned**.  ``tests/test_oracle_golden.py`` checks every function here
against fixtures under ``tests/golden/`` that were produced by running the unmodified
reference (``tests/golden/make_golden.py``) on CPU/gloo ranks.

All ranks of a sequence-parallel group are simulated inside one process: "per-rank" values
are Python lists indexed by rank, and a collective is a re-indexing of those lists.

Rank layout (yunchang convention used by ``xfuser/core/distributed/parallel_state.py:494-512``):
global SP rank ``g = ring_rank * U + ulysses_rank``; a Ulysses group is ``U`` contiguous
ranks, a ring group is ``R`` ranks strided by ``U``.  The sequence shard of rank ``g`` is the
``g``-th contiguous chunk of the global sequence.
"""
from __future__ import annotations

import numpy as np

__all__ = [
    "attention_dense",
    "attention_dense_torch_cpu",
    "merge_out_lse",
    "all_to_all_single",
    "input_all_to_all",
    "output_all_to_all",
    "combined_qkv_all_to_all",
    "preprocess_joint_kv",
    "concat_joint",
    "ring_attention",
    "usp",
    "usp_from_global",
    "KVCacheOracle",
    "long_context_attention_bshd",
    "ring_flash_attn_bshd",
    "rms_norm",
    "rope_interleaved",
    "attention_prologue",
]


# --------------------------------------------------------------------------------------
# dense attention: the back-end contract (q,k,v)[B,H,S,D] -> (out[B,H,Sq,D], lse[B,H,Sq])
# xfuser/core/distributed/attention_backend.py:492-516 (SDPA / SDPA_FLASH): scale D^-1/2,
# no dropout, optional causal mask aligned to the top-left corner.
# --------------------------------------------------------------------------------------
def attention_dense(q, k, v, scale=None, causal=False, dtype=np.float64):
    q = np.asarray(q, dtype=dtype)
    k = np.asarray(k, dtype=dtype)
    v = np.asarray(v, dtype=dtype)
    d = q.shape[-1]
    scale = float(1.0 / np.sqrt(d)) if scale is None else float(scale)  # python float: keeps `dtype`
    s = np.matmul(q, np.ascontiguousarray(np.swapaxes(k, -1, -2))) * scale
    if causal:
        sq, sk = s.shape[-2:]
        mask = np.arange(sk)[None, :] > np.arange(sq)[:, None]
        s = np.where(mask, -np.inf, s)
    m = s.max(axis=-1, keepdims=True)
    m = np.where(np.isfinite(m), m, 0.0)
    p = np.exp(s - m)
    l = p.sum(axis=-1, keepdims=True)
    out = np.matmul(p, v) / np.where(l == 0, 1.0, l)
    with np.errstate(divide="ignore"):
        lse = (m + np.log(l))[..., 0]
    return out, lse


def attention_dense_torch_cpu(q, k, v, causal=False):
    """The reference's own CPU path for the dense call, restated: its ``SDPA`` back-end is a bare
    ``F.scaled_dot_product_attention(query, key, value, dropout_p=0, is_causal=...)``
    (``xfuser/core/distributed/attention_backend.py:492-502``), which on CPU tensors runs torch's
    fused CPU kernel on all host threads.  Used for the timed CPU baseline; parity checks use
    the float64 numpy functions of this module."""
    import torch
    import torch.nn.functional as F

    return F.scaled_dot_product_attention(q, k, v, dropout_p=0.0, is_causal=causal)


def _sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def _logsigmoid(x):
    # log(sigmoid(x)) = -softplus(-x), stable on both sides
    return -np.logaddexp(0.0, -x)


def merge_out_lse(out, lse, block_out, block_lse):
    """Online-softmax merge of two partial results.

    torch ``_SDPAMerger._merge_one`` (torch/distributed/tensor/experimental/_context_parallel/
    _attention.py:158-186) and yunchang's ``update_out_and_lse`` (called from
    ``xfuser/core/long_ctx_attention/ring/ring_flash_attn.py:138``) use the same formula:
    ``out <- out - sigmoid(lse_b - lse) * (out - out_b)``; ``lse <- lse - logsigmoid(lse - lse_b)``.
    ``lse`` here is [B,H,S]; it is broadcast over D.
    """
    if out is None:
        return np.array(block_out, dtype=np.float64), np.array(block_lse, dtype=np.float64)
    lse_e = lse[..., None]
    blse_e = np.asarray(block_lse, dtype=np.float64)[..., None]
    out = out - _sigmoid(blse_e - lse_e) * (out - np.asarray(block_out, dtype=np.float64))
    lse = lse - _logsigmoid(lse - np.asarray(block_lse, dtype=np.float64))
    return out, lse


# --------------------------------------------------------------------------------------
# Ulysses all-to-all re-layouts
# --------------------------------------------------------------------------------------
def all_to_all_single(flat_per_rank):
    """Equal-split all-to-all over one group (``usp.py:87-93``): rank r receives chunk r of
    every peer's flat buffer, concatenated in peer order."""
    n = len(flat_per_rank)
    chunks = [np.split(x.reshape(-1), n) for x in flat_per_rank]
    return [np.concatenate([chunks[src][dst] for src in range(n)]) for dst in range(n)]


def input_all_to_all(x_per_rank):
    """``_ft_c_input_all_to_all`` (``usp.py:96-108``): [B,H,s,D] per rank -> [B,H/U,U*s,D]."""
    U = len(x_per_rank)
    if U <= 1:
        return list(x_per_rank)
    outs = []
    shapes = [x.shape for x in x_per_rank]
    sent = [np.ascontiguousarray(np.transpose(x, (1, 0, 2, 3))) for x in x_per_rank]
    recv = all_to_all_single(sent)
    for r in range(U):
        b, h, s, d = shapes[r]
        assert h % U == 0
        y = recv[r].reshape(U, h // U, b, -1, d)
        y = np.transpose(y, (2, 1, 0, 3, 4)).reshape(b, h // U, -1, d)
        outs.append(y)
    return outs


def output_all_to_all(x_per_rank):
    """``_ft_c_output_all_to_all`` (``usp.py:138-150``): [B,H/U,S',D] per rank -> [B,H,S'/U,D]."""
    U = len(x_per_rank)
    if U <= 1:
        return list(x_per_rank)
    sent = []
    for x in x_per_rank:
        assert x.shape[2] % U == 0
        sent.append(np.ascontiguousarray(np.transpose(x, (2, 0, 1, 3))))
    recv = all_to_all_single(sent)
    outs = []
    for r in range(U):
        b, h, s, d = x_per_rank[r].shape
        y = recv[r].reshape(U, s // U, b, -1, d)
        y = np.transpose(y, (2, 0, 3, 1, 4)).reshape(b, -1, s // U, d)
        outs.append(y)
    return outs


def combined_qkv_all_to_all(q_per_rank, k_per_rank, v_per_rank):
    """``_combined_qkv_all_to_all`` (``usp.py:111-135``): one collective for stacked q,k,v."""
    U = len(q_per_rank)
    if U <= 1:
        return list(q_per_rank), list(k_per_rank), list(v_per_rank)
    sent = []
    for q, k, v in zip(q_per_rank, k_per_rank, v_per_rank):
        b, h, s, d = q.shape
        qkv = np.stack([q, k, v], axis=0).reshape(3, b, U, h // U, s, d)
        sent.append(np.ascontiguousarray(np.transpose(qkv, (2, 0, 1, 3, 4, 5))))
    recv = all_to_all_single(sent)
    qs, ks, vs = [], [], []
    for r in range(U):
        b, h, s, d = q_per_rank[r].shape
        y = recv[r].reshape(U, 3, b, h // U, s, d)
        y = np.transpose(y, (1, 2, 3, 0, 4, 5)).reshape(3, b, h // U, -1, d)
        qs.append(y[0]); ks.append(y[1]); vs.append(y[2])
    return qs, ks, vs


def preprocess_joint_kv(joint_key, joint_value, U, ulysses_rank):
    """``_preprocess_joint_tensors`` (``usp.py:153-177``): keep this Ulysses rank's heads."""
    hp = joint_key.shape[1] // U
    sl = slice(hp * ulysses_rank, hp * (ulysses_rank + 1))
    return joint_key[:, sl], joint_value[:, sl]


def concat_joint(x, joint, strategy, axis=2):
    """``_concat_joint_tensor`` (``usp.py:179-189``)."""
    if strategy == "rear":
        return np.concatenate([x, joint], axis=axis)
    if strategy == "front":
        return np.concatenate([joint, x], axis=axis)
    raise ValueError(f"Invalid joint_strategy: {strategy}")


# --------------------------------------------------------------------------------------
# ring attention over one ring group
# --------------------------------------------------------------------------------------
def ring_attention(q_per_rank, k_per_rank, v_per_rank, joint_kv_per_rank=None, strategy=None,
                   causal=False, scale=None):
    """``ring_attn`` (``usp.py:46-74``) -> torch ``_templated_ring_attention``: at step i ring
    rank r attends to the K/V shard of ring rank (r - i) mod R; partial results are merged in
    high precision.  Joint K/V are appended once: step 0 for "front", the last step for "rear"
    (``concat_joint_tensors_decorator``, ``usp.py:218-245``).  With ``causal`` the step is
    skipped when i > r and masked on the diagonal at i == 0 (torch ``_is_causal_behavior``;
    legacy loop ``ring_flash_attn.py:104,113``)."""
    R = len(q_per_rank)
    outs, lses = [], []
    for r in range(R):
        out = lse = None
        for i in range(R):
            src = (r - i) % R
            k, v = k_per_rank[src], v_per_rank[src]
            if joint_kv_per_rank is not None:
                jk, jv = joint_kv_per_rank[r]
                if (strategy == "front" and i == 0) or (strategy == "rear" and i == R - 1):
                    k = concat_joint(k, jk, strategy)
                    v = concat_joint(v, jv, strategy)
            if causal and i > r:
                continue
            bo, bl = attention_dense(q_per_rank[r], k, v, scale=scale, causal=causal and i == 0)
            out, lse = merge_out_lse(out, lse, bo, bl)
        outs.append(out)
        lses.append(lse)
    return outs, lses


# --------------------------------------------------------------------------------------
# USP (usp.py:247-361)
# --------------------------------------------------------------------------------------
def usp(q_shards, k_shards, v_shards, U, R, joint_query=None, joint_key=None, joint_value=None,
        joint_strategy=None, combine_qkv_a2a=False):
    """Run ``USP`` for all P = U*R ranks at once.  ``*_shards[g]`` is rank g's [B,H,s,D] input;
    joint tensors are replicated [B,H,Sj,D].  Returns the list of per-rank outputs."""
    P = U * R
    assert len(q_shards) == len(k_shards) == len(v_shards) == P
    q_shards = [np.asarray(x, dtype=np.float64) for x in q_shards]
    k_shards = [np.asarray(x, dtype=np.float64) for x in k_shards]
    v_shards = [np.asarray(x, dtype=np.float64) for x in v_shards]
    joint_kv = None
    if joint_strategy:
        q_shards = [concat_joint(q, np.asarray(joint_query, dtype=np.float64), joint_strategy)
                    for q in q_shards]
        joint_kv = [
            preprocess_joint_kv(np.asarray(joint_key, dtype=np.float64),
                                np.asarray(joint_value, dtype=np.float64), U, g % U)
            for g in range(P)
        ]

    # Ulysses input all-to-all, one per Ulysses group (contiguous ranks)
    q2, k2, v2 = [None] * P, [None] * P, [None] * P
    for rr in range(R):
        grp = list(range(rr * U, (rr + 1) * U))
        qs = [q_shards[g] for g in grp]
        ks = [k_shards[g] for g in grp]
        vs = [v_shards[g] for g in grp]
        if combine_qkv_a2a and all(a.shape == b.shape == c.shape for a, b, c in zip(qs, ks, vs)):
            qo, ko, vo = combined_qkv_all_to_all(qs, ks, vs)
        else:
            qo, ko, vo = input_all_to_all(qs), input_all_to_all(ks), input_all_to_all(vs)
        for j, g in enumerate(grp):
            q2[g], k2[g], v2[g] = qo[j], ko[j], vo[j]

    # attention: one ring group per Ulysses rank (ranks strided by U)
    out = [None] * P
    for u in range(U):
        grp = list(range(u, P, U))
        jk = [joint_kv[g] for g in grp] if joint_kv is not None else None
        o, _ = ring_attention([q2[g] for g in grp], [k2[g] for g in grp], [v2[g] for g in grp],
                              joint_kv_per_rank=jk, strategy=joint_strategy)
        for j, g in enumerate(grp):
            out[g] = o[j]

    # Ulysses output all-to-all (only when U > 1, usp.py:325-353)
    if U > 1:
        for rr in range(R):
            grp = list(range(rr * U, (rr + 1) * U))
            oo = output_all_to_all([out[g] for g in grp])
            for j, g in enumerate(grp):
                out[g] = oo[j]
    return out


def usp_from_global(q, k, v, U, R, **kw):
    """Shard global [B,H,S,D] tensors contiguously over P ranks and run :func:`usp`."""
    P = U * R
    return usp(np.array_split(q, P, axis=2), np.array_split(k, P, axis=2),
               np.array_split(v, P, axis=2), U, R, **kw)


# --------------------------------------------------------------------------------------
# PipeFusion stale-KV buffer (xfuser/core/cache_manager/cache_manager.py)
# --------------------------------------------------------------------------------------
class KVCacheOracle:
    """One attention layer's persistent [K || V] buffer.

    ``update`` restates ``CacheManager.update_and_get_kv_cache`` (``cache_manager.py:64-101``)
    for the two cache types:

    * ``naive`` (``_naive_cache_update`` ``:103-135``): outside patch mode the new [K||V]
      replaces the buffer; in patch mode rows ``[start[p], start[p+1])`` along ``slice_dim`` are
      overwritten.
    * ``sp`` (``_sequence_parallel_cache_update`` ``:138-194``): with one patch the new KV is
      returned untouched and nothing is stored; outside patch mode every Ulysses-rank chunk is
      split into per-patch pieces and re-concatenated with the rank loop outermost (which
      reproduces the input order); in patch mode rows ``[U*start[p], U*start[p+1])`` are
      overwritten.  The two orders differ for U > 1: that is the reference's behaviour and is
      reproduced as is.
    """

    def __init__(self, cache_type="naive", U=1):
        assert cache_type in ("naive", "sp")
        self.cache_type = cache_type
        self.U = U
        self.buf = None

    def update(self, k, v, slice_dim, num_patches, patch_mode, patch_idx, token_start,
               token_num=None):
        new_kv = np.concatenate([k, v], axis=-1)
        if self.cache_type == "naive":
            if num_patches == 1 or not patch_mode:
                self.buf = new_kv
            else:
                self._assign(new_kv, slice_dim, token_start[patch_idx], token_start[patch_idx + 1])
            kv = self.buf
        else:
            if num_patches == 1:
                kv = new_kv
            elif not patch_mode:
                pieces = []
                splits = np.cumsum(token_num)[:-1]
                for chunk in np.array_split(new_kv, self.U, axis=slice_dim):
                    pieces.append(np.split(chunk, splits, axis=slice_dim))
                self.buf = np.concatenate(
                    [pieces[r][p] for r in range(self.U) for p in range(len(token_num))],
                    axis=slice_dim)
                kv = self.buf
            else:
                self._assign(new_kv, slice_dim, self.U * token_start[patch_idx],
                             self.U * token_start[patch_idx + 1])
                kv = self.buf
        half = kv.shape[-1] // 2
        return kv[..., :half], kv[..., half:]

    def _assign(self, new_kv, dim, start, end):
        idx = [slice(None)] * self.buf.ndim
        idx[dim] = slice(start, end)
        self.buf = self.buf.copy()
        self.buf[tuple(idx)] = new_kv


# --------------------------------------------------------------------------------------
# legacy [B,S,H,D] layer: xFuserLongContextAttention.forward + xdit_ring_flash_attn_forward
# --------------------------------------------------------------------------------------
def _seq_all_to_all_4d(x_per_rank, scatter_idx, gather_idx):
    """yunchang ``SeqAllToAll4D`` (un-vendored dependency, yunchang >= 0.6.0, no pin; used at
    ``hybrid/attn_layer.py:187-202,234``).  Published behaviour: scatter_idx=2, gather_idx=1
    turns [B, s, H, D] into [B, U*s, H/U, D] with the gathered sequence in rank order and rank
    r keeping heads [r*H/U, (r+1)*H/U); scatter_idx=1, gather_idx=2 is the inverse."""
    U = len(x_per_rank)
    if U == 1:
        return list(x_per_rank)
    outs = []
    if scatter_idx == 2 and gather_idx == 1:
        for r in range(U):
            parts = []
            for src in range(U):
                h = x_per_rank[src].shape[2] // U
                parts.append(x_per_rank[src][:, :, r * h:(r + 1) * h])
            outs.append(np.concatenate(parts, axis=1))
    elif scatter_idx == 1 and gather_idx == 2:
        for r in range(U):
            parts = []
            for src in range(U):
                s = x_per_rank[src].shape[1] // U
                parts.append(x_per_rank[src][:, r * s:(r + 1) * s])
            outs.append(np.concatenate(parts, axis=2))
    else:
        raise ValueError("unsupported scatter/gather idx")
    return outs


def ring_flash_attn_bshd(q_per_rank, k_per_rank, v_per_rank, causal=False, scale=None,
                         joint_kv_per_rank=None, joint_strategy="none"):
    """``xdit_ring_flash_attn_forward`` (``ring/ring_flash_attn.py:27-148``) over one ring group,
    tensors [B,S,H,D].  Same schedule as :func:`ring_attention`; the returned LSE is [B,H,S]
    (``:147``)."""
    t = lambda x: np.transpose(x, (0, 2, 1, 3))
    jk = None
    strat = None
    if joint_kv_per_rank is not None:
        if joint_strategy not in ("front", "rear"):
            raise ValueError(f"joint_strategy: {joint_strategy} not supprted.")
        jk = [(t(a), t(b)) for a, b in joint_kv_per_rank]
        strat = joint_strategy
    outs, lses = ring_attention([t(x) for x in q_per_rank], [t(x) for x in k_per_rank],
                                [t(x) for x in v_per_rank], joint_kv_per_rank=jk, strategy=strat,
                                causal=causal, scale=scale)
    return [t(o) for o in outs], lses


def long_context_attention_bshd(q_shards, k_shards, v_shards, U, R, joint_query=None,
                                joint_key=None, joint_value=None, joint_strategy="none",
                                causal=False, scale=None):
    """``xFuserLongContextAttention.forward`` (``hybrid/attn_layer.py:100-239``) for all ranks,
    tensors [B,s,H,D]; joint tensors [B,Sj,H,D]."""
    P = U * R
    is_joint = joint_query is not None
    if is_joint and joint_strategy not in ("front", "rear"):
        raise ValueError(f"joint_strategy: {joint_strategy} not supprted.")
    q_shards = [np.asarray(x, dtype=np.float64) for x in q_shards]
    if is_joint:
        q_shards = [concat_joint(q, np.asarray(joint_query, dtype=np.float64), joint_strategy, axis=1)
                    for q in q_shards]
    q2, k2, v2 = [None] * P, [None] * P, [None] * P
    for rr in range(R):
        grp = list(range(rr * U, (rr + 1) * U))
        for dst, src in ((q2, q_shards), (k2, k_shards), (v2, v_shards)):
            o = _seq_all_to_all_4d([np.asarray(src[g], dtype=np.float64) for g in grp], 2, 1)
            for j, g in enumerate(grp):
                dst[g] = o[j]
    out = [None] * P
    for u in range(U):
        grp = list(range(u, P, U))
        jkv = None
        if is_joint:
            hp = joint_key.shape[2] // U
            jkv = [(np.asarray(joint_key, dtype=np.float64)[:, :, u * hp:(u + 1) * hp],
                    np.asarray(joint_value, dtype=np.float64)[:, :, u * hp:(u + 1) * hp])
                   for _ in grp]
        o, _ = ring_flash_attn_bshd([q2[g] for g in grp], [k2[g] for g in grp],
                                    [v2[g] for g in grp], causal=causal, scale=scale,
                                    joint_kv_per_rank=jkv, joint_strategy=joint_strategy)
        for j, g in enumerate(grp):
            out[g] = o[j]
    for rr in range(R):
        grp = list(range(rr * U, (rr + 1) * U))
        oo = _seq_all_to_all_4d([out[g] for g in grp], 1, 2)
        for j, g in enumerate(grp):
            out[g] = oo[j]
    return out


# --------------------------------------------------------------------------------------
# attention prologue of the DiT processors (norm, rotary embedding, head split, pack)
# --------------------------------------------------------------------------------------
def round_to_storage(x, kind):
    """Round float64 values to the nearest ``"bf16"`` (8 significant bits) or ``"f16"`` (11) value, ties to
    even, returned as float64; ``None`` leaves them alone.  This is where a 16-bit module of the reference
    rounds: ``torch.nn.RMSNorm`` returns its input's dtype and the processors' rotary helper ends in
    ``.type_as(hidden_states)`` (``transformer_wan.py:99-100,120``).  Subnormals and overflow are outside
    the range these activations reach and are not modelled."""
    if kind is None:
        return np.asarray(x, dtype=np.float64)
    x = np.asarray(x, dtype=np.float64)
    if kind == "f16":
        return x.astype(np.float16).astype(np.float64)
    if kind != "bf16":
        raise ValueError(f"unknown storage type {kind!r}")
    m, e = np.frexp(x)                      # x = m * 2**e, 0.5 <= |m| < 1
    return np.ldexp(np.rint(m * 256.0), e - 8)   # np.rint rounds half to even


def storage_ulp(x, kind):
    """Spacing of ``kind`` values in the binade of ``|x|`` (for ``|x|`` below the smallest normal, that of
    the smallest normal binade)."""
    bits = {"bf16": 8, "f16": 11}[kind]
    tiny = {"bf16": 2.0 ** -126, "f16": 2.0 ** -14}[kind]
    _, e = np.frexp(np.maximum(np.abs(np.asarray(x, dtype=np.float64)), tiny))
    return np.ldexp(1.0, e - bits)


def rms_norm(x, weight, eps, group=None):
    """``torch.nn.RMSNorm`` over the last axis as the processors apply it to the q and k projections:
    ``attn.norm_q(query)`` on ``[B, s, H*D]`` in ``transformer_wan.py:99-100`` (``group=None``: one mean
    of squares over all ``H*D`` elements) or on ``[B, s, H, D]`` in ``transformer_flux.py:121-122``
    (``group=D``: one per head).  ``weight`` has ``group`` (or ``H*D``) elements."""
    x = np.asarray(x, dtype=np.float64)
    shape = x.shape
    g = shape[-1] if group is None else group
    xg = x.reshape(shape[:-1] + (shape[-1] // g, g))
    y = xg / np.sqrt(np.mean(xg * xg, axis=-1, keepdims=True) + eps)
    y = y.reshape(shape)
    w = np.asarray(weight, dtype=np.float64)
    if w.size == shape[-1]:
        return y * w
    return (y.reshape(shape[:-1] + (shape[-1] // g, g)) * w).reshape(shape)


def rope_interleaved(x, cos, sin):
    """Rotary embedding of interleaved pairs, ``transformer_wan.py:108-120``: with
    ``x1, x2 = x[..., 0::2], x[..., 1::2]``, ``out[..., 0::2] = x1*cos[..., 0::2] - x2*sin[..., 1::2]`` and
    ``out[..., 1::2] = x1*sin[..., 1::2] + x2*cos[..., 0::2]``.  ``x`` is ``[B, s, H, D]``, ``cos`` / ``sin``
    broadcast against it (``[1, s, 1, D]``)."""
    x = np.asarray(x, dtype=np.float64)
    cos = np.asarray(cos, dtype=np.float64)[..., 0::2]
    sin = np.asarray(sin, dtype=np.float64)[..., 1::2]
    x1, x2 = x[..., 0::2], x[..., 1::2]
    out = np.empty_like(x)
    out[..., 0::2] = x1 * cos - x2 * sin
    out[..., 1::2] = x1 * sin + x2 * cos
    return out


def attention_prologue(q, k, v, heads, wq=None, wk=None, eps=1e-6, per_head=False, cos=None, sin=None, U=1,
                       round_to=None):
    """What a DiT attention processor does between the q/k/v projections and the attention call
    (``transformer_wan.py:97-122,143-147``), followed by the send layout of the Ulysses all-to-all
    (``usp.py:96-108``): norm of q and k, unflatten to heads, rotary embedding of q and k, and for each
    tensor the re-layout ``[B, s, H, D] -> [U][H/U][B][s][D]``.  ``q, k, v`` are ``[B, s, H*D]``;
    ``cos`` / ``sin`` are ``[s, D]``.  Returns the three send buffers as arrays of that 5-D shape.

    ``round_to`` (``"bf16"`` / ``"f16"``) rounds to that storage type at the two places where the
    reference's 16-bit modules do: the output of the norm and the output of the rotary helper (which
    multiplies the 16-bit activations with fp32 tables, so the products and their sum are not rounded in
    between).  With ``round_to`` the result is what a 16-bit implementation is held to, element by
    element; without it, the exact real-number result."""
    outs = []
    for i, (x, w) in enumerate(((q, wq), (k, wk), (v, None))):
        x = np.asarray(x, dtype=np.float64)
        B, s, HD = x.shape
        D = HD // heads
        if w is not None:
            x = round_to_storage(rms_norm(x, w, eps, group=D if per_head else None), round_to)
        x = x.reshape(B, s, heads, D)
        if cos is not None and i < 2:  # q and k only
            x = rope_interleaved(x, np.asarray(cos)[None, :, None, :], np.asarray(sin)[None, :, None, :])
            x = round_to_storage(x, round_to)
        # [B, s, H, D] -> [U, H/U, B, s, D]
        outs.append(x.transpose(2, 0, 1, 3).reshape(U, heads // U, B, s, D))
    return tuple(outs)


# --------------------------------------------------------------------------------------------
# model boundary: zero-pad + shard at entry, gather + unpad at exit
# --------------------------------------------------------------------------------------------
def pad_and_shard_sequence(x, world, dim=1):
    """Every rank's chunk of ``x`` along ``dim`` after zero-padding that axis up to a multiple of ``world``
    (``transformer_wan.py:219-234``: ``torch.cat([x, zeros])`` then ``torch.chunk(x, world, dim)[rank]``).
    Returns ``(list of chunks, pad_amount)``."""
    x = np.asarray(x)
    n = x.shape[dim]
    pad = (world - n % world) % world
    if pad:
        shape = list(x.shape)
        shape[dim] = pad
        x = np.concatenate([x, np.zeros(shape, dtype=x.dtype)], axis=dim)
    return np.split(x, world, axis=dim), pad


def gather_and_unpad(chunks, pad, dim=-2):
    """``GroupCoordinator.all_gather(x, dim)`` (``group_coordinator.py:221-262``: rank order along ``dim``)
    followed by dropping the last ``pad`` rows (``transformer_wan.py:236-239``)."""
    x = np.concatenate([np.asarray(c) for c in chunks], axis=dim)
    n = x.shape[dim]
    return np.take(x, np.arange(n - pad), axis=dim)
