"""CPU restatement of the reference's pair-representation ops.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).  Every function is a
plain, un-fused torch transcription of the *algorithm* of one reference module
and takes that module's ``state_dict`` (same key names) as ``w``.  Arithmetic
runs in the dtype of the inputs (pass fp32 or fp64 tensors); nothing here is
tuned for speed.

Paths cited are relative to the reference project root.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import Tensor

LN_EPS = 1e-5  # nn.LayerNorm default; src/bioemu2/biomoa/ops/triangle_multiplication.py:71


def layer_norm(x: Tensor, weight: Tensor | None, bias: Tensor | None, eps: float = LN_EPS) -> Tensor:
    """Biased-variance LayerNorm over the last axis (torch.nn.LayerNorm semantics)."""
    mu = x.mean(dim=-1, keepdim=True)
    var = ((x - mu) ** 2).mean(dim=-1, keepdim=True)
    y = (x - mu) / torch.sqrt(var + eps)
    if weight is not None:
        y = y * weight
    if bias is not None:
        y = y + bias
    return y


def linear(x: Tensor, weight: Tensor, bias: Tensor | None = None) -> Tensor:
    y = x @ weight.T
    return y if bias is None else y + bias


def triangle_multiplication(x: Tensor, mask: Tensor, w: dict, mode: str, rows: slice | None = None) -> Tensor:
    """``TriangleMultiplicationFull.forward``.

    src/bioemu2/biomoa/ops/triangle_multiplication.py:86-99 (weights :62-76).
    No residual: the caller adds it (src/bioemu2/biomoa/modules/pairmixer.py:447-452).

    ``rows`` restricts the result to output rows ``i in rows`` (the projections still see the whole tensor,
    only the contraction and the output stage are cut down): the check used at sizes where the full
    contraction would take the CPU minutes.
    """
    assert mode in ("outgoing", "incoming")
    h = layer_norm(x, w["norm_in.weight"], w["norm_in.bias"])
    proj = linear(h, w["p_in.weight"]) * torch.sigmoid(linear(h, w["g_in.weight"]))
    proj = torch.where(mask.bool().unsqueeze(-1), proj, torch.zeros_like(proj))
    a, b = proj.chunk(2, dim=-1)
    if mode == "outgoing":
        t = torch.einsum("bikd,bjkd->bijd", a if rows is None else a[:, rows], b)
    else:
        t = torch.einsum("bkid,bkjd->bijd", a if rows is None else a[:, :, rows], b)
    t = layer_norm(t, w["norm_out.weight"], w["norm_out.bias"])
    h_rows = h if rows is None else h[:, rows]
    return linear(t, w["p_out.weight"]) * torch.sigmoid(linear(h_rows, w["g_out.weight"]))


def transition(x: Tensor, w: dict) -> Tensor:
    """``Transition.forward``: ``fc3(silu(fc1(LN(x))) * fc2(LN(x)))``.

    src/bioemu2/biomoa/ops/transition.py:52-76.  The LayerNorm is applied only
    when the state dict carries ``norm.*`` keys (``use_norm=True``, :44-45).
    """
    if "norm.weight" in w:
        x = layer_norm(x, w["norm.weight"], w["norm.bias"])
    return linear(F.silu(linear(x, w["fc1.weight"])) * linear(x, w["fc2.weight"]), w["fc3.weight"])


def attention_pair_bias(
    s: Tensor,
    z: Tensor,
    mask: Tensor,
    w: dict,
    num_heads: int,
    multiplicity: int = 1,
    inf: float = 1e6,
    bias: Tensor | None = None,
) -> Tensor:
    """``AttentionPairBias.forward`` (un-tiled branch).  ``bias`` ([B,H,N,N]) replaces ``proj_z(norm_z(z))`` when given
    (used to check sharded callers that assemble the bias themselves).

    src/bioemu2/biomoa/ops/attention_pair_bias.py:128-192,224-225.  The key
    mask *replaces* masked logits by ``-inf`` (finite 1e6, :183-190); the pair
    bias ``proj_z(norm_z(z))`` is shared by the ``multiplicity`` copies (:172-179).
    """
    BM, N, c_s = s.shape
    B = z.shape[0] if bias is None else bias.shape[0]
    assert BM == B * multiplicity
    H = num_heads
    dh = c_s // H
    if "norm_s.weight" in w:
        s = layer_norm(s, w["norm_s.weight"], w["norm_s.bias"])
    qkv = linear(s, w["proj_qkv.weight"])
    q, k, v = qkv.chunk(3, dim=-1)
    q = (q + w["proj_q_bias"]).view(BM, N, H, dh)
    k = k.view(BM, N, H, dh)
    v = v.view(BM, N, H, dh)
    g = torch.sigmoid(linear(s, w["proj_g.weight"]))
    if bias is None:
        zb = linear(layer_norm(z, w["norm_z.weight"], w.get("norm_z.bias")), w["proj_z.weight"])
        zb = zb.permute(0, 3, 1, 2)  # [B, H, N, N]
    else:
        zb = bias
    attn = torch.einsum("bihd,bjhd->bhij", q, k) / math.sqrt(dh)
    attn = attn.view(B, multiplicity, H, N, N) + zb.unsqueeze(1)
    key_mask = mask.bool().view(B, 1, 1, 1, N)
    attn = torch.where(key_mask, attn, torch.full_like(attn, -inf))
    attn = attn.softmax(dim=-1).view(BM, H, N, N)
    o = torch.einsum("bhij,bjhd->bihd", attn, v).reshape(BM, N, c_s)
    return linear(g * o, w["proj_o.weight"])


def attention_pair_bias_sliding_window(s: Tensor, z: Tensor, mask: Tensor, w: dict, num_heads: int,
                                       multiplicity: int = 1, inf: float = 1e6) -> Tensor:
    """``AttentionPairBiasSlidingWindow.forward``: src/bioemu2/biomoa/ops/attention_pair_bias.py:283-340.

    ``s[B*M*NW, W, c_s]`` (windows of W query atoms), ``z[B, NW, W, H, c_z]``, ``mask[B*NW, W]``.  Window ``n`` sees the
    ``H`` keys ``n*W - (H-W)/2 ...`` of its own sample; keys beyond the sequence are zero rows (the projections are
    bias-free) and count as masked (:303-318).  Masked logits are replaced by ``-inf`` after the bias is added (:331-332).
    """
    B, NW, W, H = z.shape[:4]
    folded, _, c_s = s.shape
    BM, M, dh, ctx = folded // NW, multiplicity, c_s // num_heads, (H - W) // 2
    if "norm_s.weight" in w:
        s = layer_norm(s, w["norm_s.weight"], w["norm_s.bias"])
    qkv = linear(s, w["proj_qkv.weight"])
    q = (qkv[..., :c_s] + w["proj_q_bias"]).view(folded, W, num_heads, dh)
    g = torch.sigmoid(linear(s, w["proj_g.weight"]))
    key_rows = torch.arange(NW)[:, None] * W + torch.arange(H)[None, :]          # rows of the padded sequence, [NW, H]
    kv = torch.nn.functional.pad(qkv[..., c_s:].reshape(BM, NW * W, 2 * c_s), (0, 0, ctx, ctx))[:, key_rows]
    k, v = kv.reshape(folded, H, 2, num_heads, dh).unbind(dim=2)
    mask_keys = torch.nn.functional.pad(mask.bool().reshape(B, NW * W), (ctx, ctx))[:, key_rows]   # [B, NW, H]
    zb = linear(layer_norm(z, w["norm_z.weight"], w.get("norm_z.bias")), w["proj_z.weight"]).permute(0, 1, 4, 2, 3)
    attn = torch.einsum("bihd,bjhd->bhij", q, k) / math.sqrt(dh)               # [folded, heads, W, H]
    attn = attn.view(B, M, NW, num_heads, W, H) + zb[:, None]
    attn = attn.masked_fill(~mask_keys[:, None, :, None, None, :], -inf)
    attn = attn.softmax(dim=-1).view(folded, num_heads, W, H)
    o = torch.einsum("bhij,bjhd->bihd", attn, v).reshape(folded, W, c_s)
    return linear(g * o, w["proj_o.weight"])


def outer_product_mean(m: Tensor, mask: Tensor, w: dict, i_chunk: int | None = None) -> Tensor:
    """``OuterProductMeanVanilla.forward``.

    src/bioemu2/biomoa/ops/outer_product_mean.py:45-75.  ``mask`` is ``[B,S,N]``
    (rows averaged over, :66-67) or ``[B,N]`` (divisor 1, :68-69).  ``i_chunk`` only bounds the size of the
    ``[B, i, N, c, c]`` outer-product tensor (the reference's ``tile_size`` plays the same role).
    """
    mask = mask.bool()
    c_hidden = w["proj_ab.weight"].shape[0] // 2
    mp = linear(layer_norm(m, w["norm.weight"], w["norm.bias"]), w["proj_ab.weight"])
    mp = torch.where(mask.unsqueeze(-1), mp, torch.zeros_like(mp))
    a, b = mp.chunk(2, dim=-1)
    if mask.ndim == 3:
        num_valid = mask.any(dim=-1).sum(dim=1).clamp(min=1).to(m.dtype)
    else:
        num_valid = torch.ones(m.shape[0], dtype=m.dtype)
    n = m.shape[2]
    step = n if i_chunk is None else i_chunk
    outs = []
    for i0 in range(0, n, step):
        z = torch.einsum("bsic,bsjd->bijcd", a[:, :, i0:i0 + step], b)
        z = z.reshape(*z.shape[:3], c_hidden * c_hidden) / num_valid[:, None, None, None]
        outs.append(linear(z, w["proj_o.weight"], w["proj_o.bias"]))
    return torch.cat(outs, dim=1)


def _sub(w: dict, prefix: str) -> dict:
    p = prefix + "."
    return {k[len(p):]: v for k, v in w.items() if k.startswith(p)}


def pairmixer_layer(z: Tensor, pair_mask: Tensor, w: dict) -> Tensor:
    """``PairMixerLayer.forward`` in eval mode (dropout is the identity).

    src/bioemu2/biomoa/modules/pairmixer.py:430-456; ``s`` passes through
    unchanged and is therefore not an argument here.
    """
    z = z + triangle_multiplication(z, pair_mask, _sub(w, "tri_mul_out"), "outgoing")
    z = z + triangle_multiplication(z, pair_mask, _sub(w, "tri_mul_in"), "incoming")
    z = z + transition(z, _sub(w, "transition_z"))
    return z


def pair_weighted_averaging(m: Tensor, z: Tensor, mask: Tensor, w: dict, num_heads: int = 8, inf: float = 1e6) -> Tensor:
    """``PairWeightedAveraging.forward`` (un-chunked branch).

    src/bioemu2/biomoa/ops/pair_weighted_averaging.py:121-153: weights ``softmax_j(proj_z(norm_z(z))[i, j, h])`` with
    masked pairs REPLACED by ``-inf`` (finite 1e6, :141), values ``proj_m(norm_m(m))``, gate ``sigmoid(proj_g(norm_m(m)))``,
    ``out[s, i] = proj_o(gate * sum_j w[h, i, j] v[s, j, h, :])``.  ``m[B,S,N,c_m]``, ``z[B,N,N,c_z]``, ``mask[B,N,N]``.
    """
    B, S, N, _ = m.shape
    H = num_heads
    mn = layer_norm(m, w["norm_m.weight"], w["norm_m.bias"])
    v = linear(mn, w["proj_m.weight"])
    c_h = v.shape[-1] // H
    v = v.view(B, S, N, H, c_h)
    b = linear(layer_norm(z, w["norm_z.weight"], w.get("norm_z.bias")), w["proj_z.weight"]).permute(0, 3, 1, 2)
    b = torch.where(mask.bool()[:, None], b, torch.full_like(b, -inf))
    wts = b.softmax(dim=-1)                                   # [B, H, i, j]
    g = torch.sigmoid(linear(mn, w["proj_g.weight"]))
    o = torch.einsum("bhij,bsjhd->bsihd", wts, v).reshape(B, S, N, H * c_h)
    return linear(g * o, w["proj_o.weight"])


def pairmixer_msa_layer(z: Tensor, m: Tensor, pair_mask: Tensor, msa_mask: Tensor, w: dict):
    """``PairMixerMSALayer.forward`` in eval mode: returns ``(z, m)`` (``s`` passes through).

    src/bioemu2/biomoa/modules/pairmixer.py:738-757: ``m += PWA(m, z); m += T(m); z += OPM(m); z += TriMul_out(z);
    z += TriMul_in(z); z += T(z)``.
    """
    m = m + pair_weighted_averaging(m, z, pair_mask, _sub(w, "pair_weighted_averaging"))
    m = m + transition(m, _sub(w, "msa_transition"))
    z = z + outer_product_mean(m, msa_mask, _sub(w, "outer_product_mean"))
    z = z + triangle_multiplication(z, pair_mask, _sub(w, "tri_mul_out"), "outgoing")
    z = z + triangle_multiplication(z, pair_mask, _sub(w, "tri_mul_in"), "incoming")
    z = z + transition(z, _sub(w, "z_transition"))
    return z, m


def pairmixer_module(z: Tensor, pair_mask: Tensor, w: dict, num_blocks: int) -> Tensor:
    """``PairMixerModule.forward``: src/bioemu2/biomoa/modules/pairmixer.py:368-370."""
    for i in range(num_blocks):
        z = pairmixer_layer(z, pair_mask, _sub(w, f"layers.{i}"))
    return z


def pairwise_conditioning(z_trunk: Tensor, rel_pos_feats: Tensor, w: dict, num_transitions: int = 2) -> Tensor:
    """``PairwiseConditioning.forward``: src/bioemu2/biomoa/modules/diffusion.py:526-534.

    ``Linear(LN(cat(z_trunk, rel_pos_feats)))`` (:493-494, no bias), then ``z = T(z) + z`` per transition.
    """
    z = torch.cat((z_trunk, rel_pos_feats), dim=-1)
    z = linear(layer_norm(z, w["dim_pairwise_init_proj.0.weight"], w["dim_pairwise_init_proj.0.bias"]),
               w["dim_pairwise_init_proj.1.weight"])
    for i in range(num_transitions):
        z = transition(z, _sub(w, f"transitions.{i}")) + z
    return z


def pairmixer_msa_module(z: Tensor, emb: Tensor, feats: dict, w: dict, blocks: int, use_paired_feature: bool = True) -> Tensor:
    """``PairMixerMSAModule.forward`` with ``s=None``: src/bioemu2/biomoa/modules/pairmixer.py:582-612.

    ``m = msa_proj(cat(msa, has_deletion, deletion_value[, msa_paired])) + s_proj(emb)[:, None]`` (:590-599), then the MSA
    layers; only the pair tensor leaves the module.
    """
    dt = w["msa_proj.weight"].dtype
    cols = [feats["msa"].to(dt), feats["has_deletion"].to(dt)[..., None], feats["deletion_value"].to(dt)[..., None]]
    if use_paired_feature:
        cols.append(feats["msa_paired"].to(dt)[..., None])
    m = linear(torch.cat(cols, dim=-1), w["msa_proj.weight"]) + linear(emb, w["s_proj.weight"])[:, None]
    tok = feats["token_pad_mask"].bool()
    pair_mask = tok[:, :, None] & tok[:, None, :]
    for i in range(blocks):
        z, m = pairmixer_msa_layer(z, m, pair_mask, feats["msa_mask"], _sub(w, f"layers.{i}"))
    return z


def sequence_trunk(s_inputs: Tensor, pair_terms: Tensor, feats: dict, w: dict, *, recycles: int, msa_blocks: int,
                   num_blocks: int, unconditional: bool = False, use_paired_feature: bool = True):
    """``PairMixerSequenceEmbedder.forward``: src/bioemu2/biomoa/modules/pairmixer.py:231-299.

    ``pair_terms`` is the sum of what the feature encoders add to the pair initialisation (relative positions, token
    bonds, optional conditioning; :240-256): they are input featurisation, not part of the hot path, and enter as data.
    """
    s_init = linear(s_inputs, w["s_init.weight"])
    z_init = linear(s_inputs, w["z_init_1.weight"])[:, :, None] + linear(s_inputs, w["z_init_2.weight"])[:, None, :]
    z_init = z_init + pair_terms
    if unconditional:  # :262-270
        zn = layer_norm(z_init, w["z_norm.weight"], w["z_norm.bias"])
        return s_init, z_init + transition(zn, _sub(w, "uncond_transition"))
    tok = feats["token_pad_mask"].bool()
    pair_mask = tok[:, :, None] & tok[:, None, :]
    s, z = torch.zeros_like(s_init), torch.zeros_like(z_init)
    for _ in range(recycles + 1):  # :272-297
        s = s_init + linear(layer_norm(s, w["s_norm.weight"], w["s_norm.bias"]), w["s_recycle.weight"])
        z = z_init + linear(layer_norm(z, w["z_norm.weight"], w["z_norm.bias"]), w["z_recycle.weight"])
        z = pairmixer_msa_module(z, s_inputs, feats, _sub(w, "msa_module"), msa_blocks, use_paired_feature)
        z = pairmixer_module(z, pair_mask, _sub(w, "pairmixer_module"), num_blocks)  # s passes through (:368-370)
    return s, z


def triangle_attention(x: Tensor, mask: Tensor, w: dict, num_heads: int, ending: bool, inf: float = 1e6,
                       row_chunk: int | None = None, lines: slice | None = None) -> Tensor:
    """Triangle self-attention around the starting (or ending) node.

    NOT IN THE REFERENCE -- parity unpinned.  The reference removed this op
    (src/bioemu2/biomoa/modules/pairmixer.py:459-462), so this is the published
    AlphaFold-2 algorithm (Jumper et al. 2021, suppl. alg. 13/14) written with
    the reference's pair-bias-attention conventions: bias-free projections, LN
    eps 1e-5, finite ``inf`` replacing masked logits, and a gating projection
    with a bias (initialised to 1 by the module).

    ``x[B,N,N,D]``, ``mask[B,N,N]``.  Starting node: row ``i`` attends from
    ``j`` to ``k`` with logits ``q[i,j]·k[i,k]/sqrt(dh) + bias[j,k]`` and keys
    masked by ``mask[i,k]``.  Ending node is the same on the transposed pair
    tensor.  ``lines`` restricts the result to attention lines ``i in lines``
    (rows of the output for the starting node, columns for the ending node);
    the triangle bias still comes from the whole tensor.
    """
    if ending:
        x = x.transpose(1, 2)
        mask = mask.transpose(1, 2)
    B, N, _, D = x.shape
    H = num_heads
    h = layer_norm(x, w["layer_norm.weight"], w["layer_norm.bias"])
    dh = w["linear_q.weight"].shape[0] // H
    q = linear(h, w["linear_q.weight"]).view(B, N, N, H, dh)
    k = linear(h, w["linear_k.weight"]).view(B, N, N, H, dh)
    v = linear(h, w["linear_v.weight"]).view(B, N, N, H, dh)
    tri_bias = linear(h, w["linear_b.weight"]).permute(0, 3, 1, 2)  # [B,H,j,k]
    g = torch.sigmoid(linear(h, w["linear_g.weight"], w["linear_g.bias"]))
    # rows i are independent; row_chunk only bounds the size of the [B, rows, H, N, N] logits tensor
    lo, hi, _ = (lines or slice(None)).indices(N)
    step = (hi - lo) if row_chunk is None else row_chunk
    o_rows = []
    for i0 in range(lo, hi, step):
        sl = slice(i0, min(i0 + step, hi))
        logits = torch.einsum("bijhd,bikhd->bihjk", q[:, sl], k[:, sl]) / math.sqrt(dh)
        logits = logits + tri_bias.unsqueeze(1)
        key_mask = mask[:, sl].bool().view(B, -1, 1, 1, N)
        logits = torch.where(key_mask, logits, torch.full_like(logits, -inf))
        p = logits.softmax(dim=-1)
        o_rows.append(torch.einsum("bihjk,bikhd->bijhd", p, v[:, sl]))
    o = torch.cat(o_rows, dim=1).reshape(B, hi - lo, N, H * dh)
    out = linear(g[:, lo:hi] * o, w["linear_o.weight"])
    if ending:
        out = out.transpose(1, 2)
    return out


def pairformer_block(s: Tensor, z: Tensor, token_mask: Tensor, w: dict, *, tri_heads: int = 4, apb_heads: int = 16,
                     row_chunk: int | None = None):
    """The composite block the benchmark configs describe.

    Pair track: triangle multiplication out/in, triangle attention start/end,
    pair transition; single track: pair-bias attention and a transition, each
    with a residual.  The reference's own block stops after the pair
    transition (src/bioemu2/biomoa/modules/pairmixer.py:430-456); the attention
    parts are assembled from ``AttentionPairBias`` and the unpinned triangle
    attention above.
    """
    pair_mask = token_mask[:, :, None] & token_mask[:, None, :]
    z = z + triangle_multiplication(z, pair_mask, _sub(w, "tri_mul_out"), "outgoing")
    z = z + triangle_multiplication(z, pair_mask, _sub(w, "tri_mul_in"), "incoming")
    z = z + triangle_attention(z, pair_mask, _sub(w, "tri_att_start"), tri_heads, ending=False, row_chunk=row_chunk)
    z = z + triangle_attention(z, pair_mask, _sub(w, "tri_att_end"), tri_heads, ending=True, row_chunk=row_chunk)
    z = z + transition(z, _sub(w, "transition_z"))
    s = s + attention_pair_bias(s, z, token_mask, _sub(w, "attention"), apb_heads)
    s = s + transition(s, _sub(w, "transition_s"))
    return s, z


def conditioned_transformer_layer(
    x: Tensor, pairs: Tensor, c: Tensor, mask: Tensor, w: dict, num_heads: int,
    multiplicity: int = 1, lns_scale: float = 1.0,
) -> Tensor:
    """``ConditionedTransformerLayer.forward`` (full-attention token block).

    src/bioemu2/biomoa/modules/transformer.py:317-353 with ``ada_ln`` :26-41:
    ``x += gamma1 * APB(lns*((1+alpha1)*LN(x)+beta1)); x += gamma2 * T(lns*(...))``.
    State-dict keys: ``cond.0.{weight,bias}`` (LayerNorm), ``cond.2.{weight,bias}``
    (Linear), ``attention.pair_bias_attn.*``, ``transition.*``.
    """
    cc = layer_norm(c, w["cond.0.weight"], w["cond.0.bias"])
    cc = linear(F.silu(cc), w["cond.2.weight"], w["cond.2.bias"])
    a1, b1, g1, a2, b2, g2 = cc.chunk(6, dim=-1)
    t = lns_scale * (layer_norm(x, None, None) * (1 + a1) + b1)
    if pairs.ndim == 5:
        # windowed atom attention (SlidingWindowAttentionLayer.forward, transformer.py:198-229): atoms folded into
        # query windows, ``pairs[B, NW, W, H, c]``, ``mask[B, N]``; keys ``attention.attention_layer.pair_bias_attn.*``
        BM, N, D = x.shape
        B, NW, W = pairs.shape[:3]
        h = attention_pair_bias_sliding_window(
            t.reshape(BM * NW, W, D), pairs, mask.reshape(B * NW, W),
            _sub(w, "attention.attention_layer.pair_bias_attn"), num_heads, multiplicity).reshape(BM, N, D)
    else:
        h = attention_pair_bias(t, pairs, mask, _sub(w, "attention.pair_bias_attn"), num_heads, multiplicity)
    x = x + g1 * h
    h = transition(lns_scale * (layer_norm(x, None, None) * (1 + a2) + b2), _sub(w, "transition"))
    return x + g2 * h
