"""The sequence trunk around the PairMixer blocks, with the reference's contracts
(src/bioemu2/biomoa/modules/pairmixer.py:23-299 ``PairMixerSequenceEmbedder``, :459-612 ``PairMixerMSAModule``).

What runs here is the HBM-bound glue the blocks sit in: the pair initialisation (an outer sum of two projections of
the input embedding plus the pair terms of the feature encoders), the recycling update
``z_init + z_recycle(z_norm(z))``, the MSA embedding, and the loop over the MSA and PairMixer blocks.  The feature
encoders themselves (relative positions, token bonds, contact / method conditioning) are input featurisation: they run
once per system on tiny inputs and stay whatever ``nn.Module`` the caller supplies.
"""
from __future__ import annotations

import torch
import torch.nn as nn
from torch import Tensor

from . import functional as F
from .pairmixer import PairMixerModule, PairMixerMSALayer
from .transition import Transition

NUM_TOKENS = 33  # residue-token vocabulary of the reference (src/bioemu2/data_interface/const.py)


class _PaddedLinear:
    """bf16 copy of a bias-free ``nn.Linear`` weight with the input width padded to a multiple of 8 (the tensor-map
    rows must be 16-byte multiples); rebuilt when the parameter changes."""

    def __init__(self, linear: nn.Linear):
        self.linear = linear
        self.w: Tensor | None = None
        self.version = -1

    def weight(self) -> Tensor:
        p = self.linear.weight
        if self.w is None or self.version != p._version or self.w.device != p.device:
            k = p.shape[1]
            kp = (k + 7) // 8 * 8
            w = torch.zeros(p.shape[0], kp, dtype=torch.bfloat16, device=p.device)
            w[:, :k] = p.detach()
            self.w, self.version = w, p._version
        return self.w

    def operand(self, x: Tensor) -> Tensor:
        """``x[..., k]`` as a zero-padded bf16 GEMM operand ``[..., kp]``."""
        k = x.shape[-1]
        kp = (k + 7) // 8 * 8
        if kp == k:
            return x.to(torch.bfloat16).contiguous()
        xb = torch.zeros(x.shape[:-1] + (kp,), dtype=torch.bfloat16, device=x.device)
        xb[..., :k] = x
        return xb

    def __call__(self, xb: Tensor) -> Tensor:
        return F.linear_bf16(xb, self.weight(), out_dtype=torch.float32)


class PairMixerMSAModule(nn.Module):
    """``m = msa_proj(cat(msa, has_deletion, deletion_value[, msa_paired])) + s_proj(emb)[:, None]``, then the MSA
    blocks; returns ``(s, z)`` with ``s`` passed through (pairmixer.py:582-612).  Keywords that pick among the
    reference's kernel variants, tile sizes and dropout rates are accepted and ignored (inference only)."""

    def __init__(self, token_s: int, msa_s: int, token_z: int, s_input_dim: int, msa_blocks: int,
                 msa_dropout: float = 0.0, z_dropout: float = 0.0, use_paired_feature: bool = False,
                 trimul_variant=None, trimul_tile_size: int | None = None, transition_chunk_size: int | None = None,
                 opm_variant=None, opm_tile_size: int | None = None, pwa_chunk_heads: bool = False,
                 opm_matmul_precision: str | None = None, trimul_matmul_precision: str | None = None,
                 num_tokens: int = NUM_TOKENS) -> None:
        super().__init__()
        self.msa_blocks = msa_blocks
        self.msa_dropout, self.z_dropout = msa_dropout, z_dropout
        self.use_paired_feature = use_paired_feature
        self.pwa_chunk_heads = pwa_chunk_heads
        self.s_proj = nn.Linear(s_input_dim, msa_s, bias=False)
        self.msa_proj = nn.Linear(num_tokens + 2 + int(use_paired_feature), msa_s, bias=False)
        self.layers = nn.ModuleList(
            [PairMixerMSALayer(token_s, msa_s, token_z, msa_dropout, z_dropout,
                               transition_chunk_size=transition_chunk_size, opm_tile_size=opm_tile_size)
             for _ in range(msa_blocks)])
        self._s_proj, self._msa_proj = _PaddedLinear(self.s_proj), _PaddedLinear(self.msa_proj)

    def forward(self, s: Tensor | None, z: Tensor, emb: Tensor, msa: Tensor, msa_mask: Tensor, has_deletion: Tensor,
                deletion_value: Tensor, msa_paired: Tensor, token_pad_mask: Tensor) -> tuple[Tensor | None, Tensor]:
        if self.training:
            raise RuntimeError("bioemu2_b200 modules are inference-only: call .eval()")
        m = self.embed_msa(emb, msa, has_deletion, deletion_value, msa_paired)
        tok = token_pad_mask.bool()
        token_mask = tok.unsqueeze(-1) & tok.unsqueeze(-2)
        for layer in self.layers:
            s, z, m = layer(s, z, m, token_mask, msa_mask, False)
        return s, z

    def embed_msa(self, emb: Tensor, msa: Tensor, has_deletion: Tensor, deletion_value: Tensor, msa_paired: Tensor,
                  tokens: slice | None = None) -> Tensor:
        """``msa_proj(cat(msa, has_deletion, deletion_value[, msa_paired])) + s_proj(emb)[:, None]`` as fp32
        ``[B, R, T, msa_s]`` (pairmixer.py:590-599).  ``tokens`` selects the token block a context-parallel rank holds:
        the MSA tensors then cover that block only, ``emb`` stays whole."""
        B, R, T = msa.shape[:3]
        width = self.msa_proj.in_features
        # the MSA features as one zero-padded bf16 operand (one-hot rows and 0/1 flags are exact in bf16)
        feat = torch.zeros(B, R, T, (width + 7) // 8 * 8, dtype=torch.bfloat16, device=msa.device)
        nt = msa.shape[-1]
        feat[..., :nt] = msa
        feat[..., nt] = has_deletion
        feat[..., nt + 1] = deletion_value
        if self.use_paired_feature:
            feat[..., nt + 2] = msa_paired
        if nt + 2 + int(self.use_paired_feature) != width:
            raise ValueError(f"msa has {nt} feature columns, msa_proj expects {width - 2 - int(self.use_paired_feature)}")
        m = self._msa_proj(feat)                                    # fp32 [B, R, T, msa_s]
        e = self._s_proj(self._s_proj.operand(emb))                 # fp32 [B, tokens, msa_s]
        if tokens is not None:
            e = e[:, tokens].contiguous()
        for b in range(B):
            F.add_rows(m[b], e[b], out=m[b])                        # broadcast over the MSA rows
        return m


class PairMixerSequenceEmbedder(nn.Module):
    """The recycling trunk (pairmixer.py:202-299).  ``forward(s_inputs, feats, num_steps_recycle, unconditional)`` with
    the reference's feature dictionary.

    The feature encoders are not rebuilt here: ``rel_pos``, ``token_bonds``, ``contact_conditioning`` and
    ``method_conditioning`` are ``None`` until the caller assigns modules to them (``swap_into`` / ``to_b200`` move the
    reference's own encoders across); each one present is called exactly as the reference calls it (:234-256).
    ``feats["pair_init_terms"]``, if present, is added to the pair initialisation as well - the way to supply
    precomputed encoder outputs.  Keywords for kernel variants, tiling, precision overrides and dropout are accepted
    and ignored (inference only).
    """

    def __init__(self, token_s: int, token_z: int, s_input_dim: int, msa_s: int = 64, msa_blocks: int = 4,
                 msa_dropout: float = 0.15, z_dropout: float = 0.25, num_blocks: int = 48, dropout: float = 0.0,
                 trimul_variant=None, opm_variant=None, tiling_cfg: dict | None = None, relpos_cfg: dict | None = None,
                 precision_cfg: dict | None = None, use_contact_conditioning: bool = False,
                 use_method_conditioning: bool = False, embed_method_into_pairs: bool = False,
                 use_paired_feature: bool = True, use_unconditional_branch: bool = False,
                 num_tokens: int = NUM_TOKENS) -> None:
        super().__init__()
        if token_s % 8 or token_z != 128:
            raise ValueError("bioemu2_b200.PairMixerSequenceEmbedder needs token_z == 128 and token_s a multiple of 8")
        self.token_s, self.token_z, self.s_input_dim = token_s, token_z, s_input_dim
        self.use_contact_conditioning = use_contact_conditioning
        self.use_method_conditioning = use_method_conditioning
        self.use_unconditional_branch = use_unconditional_branch
        self.s_init = nn.Linear(s_input_dim, token_s, bias=False)
        self.z_init_1 = nn.Linear(s_input_dim, token_z, bias=False)
        self.z_init_2 = nn.Linear(s_input_dim, token_z, bias=False)
        self.rel_pos: nn.Module | None = None
        self.token_bonds: nn.Module | None = None
        self.contact_conditioning: nn.Module | None = None
        self.method_conditioning: nn.Module | None = None
        self.msa_module = PairMixerMSAModule(token_s, msa_s, token_z, s_input_dim, msa_blocks, msa_dropout, z_dropout,
                                             use_paired_feature=use_paired_feature, num_tokens=num_tokens)
        self.pairmixer_module = PairMixerModule(token_s, token_z, num_blocks, dropout)
        self.s_recycle = nn.Linear(token_s, token_s, bias=False)
        self.z_recycle = nn.Linear(token_z, token_z, bias=False)
        self.s_norm = nn.LayerNorm(token_s)
        self.z_norm = nn.LayerNorm(token_z)
        if use_unconditional_branch:
            self.uncond_transition = Transition(dim=token_z, hidden=token_z * 4)
        self._lin = {n: _PaddedLinear(getattr(self, n)) for n in ("s_init", "z_init_1", "z_init_2", "s_recycle", "z_recycle")}

    # ------------------------------------------------------------------------------------------ pieces
    def initial_embeddings(self, s_inputs: Tensor, feats: dict) -> tuple[Tensor, Tensor]:
        """``s_init`` and ``z_init`` (pairmixer.py:231-256): three small GEMMs and one write of the pair tensor."""
        xb = self._lin["s_init"].operand(s_inputs)
        s_init = self._lin["s_init"](xb)
        a, c = self._lin["z_init_1"](xb), self._lin["z_init_2"](xb)
        extra = None

        def add(t: Tensor | None) -> None:
            nonlocal extra
            if t is not None:
                extra = t.float() if extra is None else extra + t.float()

        if self.method_conditioning is not None and self.use_method_conditioning:
            single_method, pair_method = self.method_conditioning(method_feature=feats["method_feature"],
                                                                  token_pad_mask=feats["token_pad_mask"])
            s_init = F.add_rows(s_init, single_method.float().expand_as(s_init).contiguous())
            add(pair_method)
        if self.rel_pos is not None:
            add(self.rel_pos(asym_id=feats["asym_id"], entity_id=feats["entity_id"],
                             residue_index=feats["residue_index"], sym_id=feats["sym_id"]))
        if self.token_bonds is not None:
            add(self.token_bonds(feats["token_bonds"]))
        if self.contact_conditioning is not None and self.use_contact_conditioning:
            add(self.contact_conditioning(contact_conditioning=feats["contact_conditioning"],
                                          contact_threshold=feats["contact_threshold"],
                                          token_pad_mask=feats["token_pad_mask"]))
        add(feats.get("pair_init_terms"))
        if extra is not None:
            extra = extra.expand(a.shape[0], a.shape[1], c.shape[1], a.shape[2])
        return s_init, F.pair_outer_sum(a, c, extra)

    def _recycle(self, x: Tensor, x_init: Tensor, norm: nn.LayerNorm, name: str) -> Tensor:
        """``x_init + recycle(norm(x))`` (pairmixer.py:282-283): LayerNorm pass, then a GEMM that adds ``x_init``."""
        xn = F.rows_to_bf16(x, norm.weight, norm.bias)
        return F.linear_bf16(xn, self._lin[name].weight(), residual=x_init, out_dtype=torch.float32)

    # ------------------------------------------------------------------------------------------ forward
    def forward(self, s_inputs: Tensor, feats: dict, num_steps_recycle: int = 0,
                unconditional: bool = False) -> tuple[Tensor, Tensor]:
        if self.training:
            raise RuntimeError("bioemu2_b200 modules are inference-only: call .eval()")
        if not unconditional and num_steps_recycle < 0:
            raise ValueError("num_steps_recycle must be non-negative; use unconditional=True.")
        s_init, z_init = self.initial_embeddings(s_inputs, feats)
        if unconditional:
            if not self.use_unconditional_branch:
                raise ValueError("Passing unconditional=True at inference time requires use_unconditional_branch=True "
                                 "at __init__")
            zn = F.rows_to_bf16(z_init, self.z_norm.weight, self.z_norm.bias)
            return s_init, F.add_rows(z_init, self.uncond_transition(zn))
        mask = feats["token_pad_mask"].bool()
        pair_mask = mask.unsqueeze(-1) & mask.unsqueeze(-2)
        s, z = torch.zeros_like(s_init), torch.zeros_like(z_init)
        for _ in range(num_steps_recycle + 1):
            s = self._recycle(s, s_init, self.s_norm, "s_recycle")
            z = self._recycle(z, z_init, self.z_norm, "z_recycle")
            _, z = self.msa_module(None, z, s_inputs, feats["msa"], feats["msa_mask"], feats["has_deletion"],
                                   feats["deletion_value"], feats["msa_paired"], feats["token_pad_mask"])
            s, z = self.pairmixer_module(s, z, pair_mask=pair_mask)
        return s, z
