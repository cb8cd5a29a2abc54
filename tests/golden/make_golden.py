"""Generate ``golden_fp32.pt`` by running the REFERENCE's own torch modules.

Run in a container that has the reference checkout (it is imported in place
through ``oracle.reference_shim``; nothing is copied):

    python tests/golden/make_golden.py

For each case in ``cases.py`` the reference module is constructed, the seeded
weights are loaded through ``load_state_dict`` (strict), and the fp32 forward
output is stored together with a checksum of the inputs.
"""
from __future__ import annotations

import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import cases as C  # noqa: E402
from oracle import reference_shim  # noqa: E402


def run_reference(case: dict) -> torch.Tensor:
    R = reference_shim.modules()
    kind = case["kind"]
    w = case["w"]
    with torch.no_grad():
        if kind == "trimul":
            cls = R.TriangleMultiplicationOutgoing if case["mode"] == "outgoing" else R.TriangleMultiplicationIncoming
            mod = cls(dim=case["x"].shape[-1]).eval()
            mod.load_state_dict(w, strict=True)
            return mod(case["x"], case["mask"])
        if kind == "transition":
            mod = R.Transition(case["x"].shape[-1], case["hidden"], use_norm=case["use_norm"]).eval()
            mod.load_state_dict(w, strict=True)
            return mod(case["x"])
        if kind == "apb":
            mod = R.AttentionPairBias(case["s"].shape[-1], case["z"].shape[-1], case["heads"],
                                      initial_norm=case["initial_norm"]).eval()
            mod.load_state_dict(w, strict=True)
            return mod(case["s"], case["z"], case["mask"], multiplicity=case["M"])
        if kind == "opm":
            mod = R.OuterProductMeanVanilla(case["m"].shape[-1], case["c_hidden"], case["c_out"]).eval()
            mod.load_state_dict(w, strict=True)
            return mod(case["m"], case["mask"])
        if kind == "pairmixer":
            mod = R.PairMixerLayer(384, case["z"].shape[-1], trimul_variant="full").eval()
            mod.load_state_dict(w, strict=True)
            s = torch.zeros(1, case["z"].shape[1], 384)
            return mod(s, case["z"], case["pair_mask"])[1]
        if kind == "cond_layer":
            from bioemu2.biomoa.modules.transformer import ConditionedTransformerLayer

            window = case.get("window")
            mod = ConditionedTransformerLayer(
                dim=case["x"].shape[-1], dim_pairwise=case["z"].shape[-1], dim_cond=case["c"].shape[-1],
                heads=case["heads"], transition_hidden=case["hidden"], lns_scale=case["lns_scale"],
                is_sliding_window=window is not None, window_queries=window[0] if window else None,
                window_keys=window[1] if window else None,
            ).eval()
            mod.load_state_dict(w, strict=True)
            return mod(case["x"], case["z"], case["c"], case["mask"], multiplicity=case["M"])
        if kind == "pwa":
            from bioemu2.biomoa.ops.pair_weighted_averaging import PairWeightedAveraging

            mod = PairWeightedAveraging(c_m=case["m"].shape[-1], c_z=case["z"].shape[-1], c_h=32, num_heads=8).eval()
            mod.load_state_dict(w, strict=True)
            return mod(case["m"], case["z"], case["mask"])
        if kind == "msa_layer":
            from bioemu2.biomoa.modules.pairmixer import PairMixerMSALayer

            mod = PairMixerMSALayer(token_s=384, msa_s=64, token_z=128, msa_dropout=0.0, z_dropout=0.0,
                                    trimul_variant="full").eval()
            mod.load_state_dict(w, strict=True)
            s = torch.zeros(1, case["z"].shape[1], 384)
            _, z, m = mod(s, case["z"], case["m"], case["pair_mask"], case["msa_mask"])
            return torch.cat([z.flatten(), m.flatten()])   # both updated tensors, pair first
        if kind == "pairwise_conditioning":
            from bioemu2.biomoa.modules.diffusion import PairwiseConditioning

            mod = PairwiseConditioning(token_z=128, dim_token_rel_pos_feats=128).eval()
            mod.load_state_dict(w, strict=True)
            return mod(case["z"], case["rel"])
        if kind == "msa_module":
            from bioemu2.biomoa.modules.pairmixer import PairMixerMSAModule

            f = case["feats"]
            mod = PairMixerMSAModule(token_s=384, msa_s=64, token_z=128, s_input_dim=case["emb"].shape[-1],
                                     msa_blocks=case["blocks"], msa_dropout=0.0, z_dropout=0.0, use_paired_feature=True,
                                     trimul_variant="full").eval()
            mod.load_state_dict(w, strict=True)
            return mod(None, case["z"], case["emb"], f["msa"], f["msa_mask"], f["has_deletion"], f["deletion_value"],
                       f["msa_paired"], f["token_pad_mask"])[1]
        if kind == "sequence_trunk":
            from bioemu2.biomoa.modules.pairmixer import PairMixerSequenceEmbedder

            class Fixed(torch.nn.Module):  # stands in for a feature encoder: returns a fixed tensor
                def __init__(self, t):
                    super().__init__()
                    self.t = t

                def forward(self, *args, **kwargs):
                    return self.t

            mod = PairMixerSequenceEmbedder(
                token_s=384, token_z=128, s_input_dim=case["s_inputs"].shape[-1], msa_s=64, msa_blocks=case["msa_blocks"],
                msa_dropout=0.0, z_dropout=0.0, num_blocks=case["num_blocks"], trimul_variant="full", opm_variant="vanilla",
                use_contact_conditioning=False, use_method_conditioning=False, use_paired_feature=True,
                use_unconditional_branch=True).eval()
            missing, unexpected = mod.load_state_dict(w, strict=False)
            assert not unexpected and all(k.startswith(("rel_pos.", "token_bonds.")) for k in missing), (missing, unexpected)
            # The feature encoders are input featurisation outside the path: their sum enters as the fixed `pair_terms`.
            mod.rel_pos = Fixed(case["pair_terms"])
            mod.token_bonds = Fixed(torch.zeros_like(case["pair_terms"]))
            feats = dict(case["feats"], asym_id=None, entity_id=None, residue_index=None, sym_id=None, token_bonds=None)
            s, z = mod(case["s_inputs"], feats, num_steps_recycle=case["recycles"], unconditional=case["unconditional"])
            return torch.cat([z.flatten(), s.flatten()])   # pair tensor first, then the single representation
        if kind == "window_apb":
            from bioemu2.biomoa.ops.attention_pair_bias import AttentionPairBiasSlidingWindow

            mod = AttentionPairBiasSlidingWindow(case["s"].shape[-1], case["z"].shape[-1], case["heads"],
                                                 window_queries=case["W"], window_keys=case["Hk"]).eval()
            mod.load_state_dict(w, strict=True)
            return mod(case["s"], case["z"], case["mask"], multiplicity=case["M"])
    raise KeyError(kind)


def main() -> None:
    torch.set_num_threads(2)  # fixed reduction order, as the reference's tests/conftest.py:5-10
    out = {}
    for name, make in C.CASES.items():
        case = make()
        y = run_reference(case)
        out[name] = {"output": y.float().contiguous(), "input_checksum": C.checksum(C.case_tensors(case))}
        print(f"{name:28s} out {tuple(y.shape)} absmax {float(y.abs().max()):.4f}")
    torch.save(out, C.GOLDEN_PATH)
    print("wrote", C.GOLDEN_PATH, os.path.getsize(C.GOLDEN_PATH), "bytes")


if __name__ == "__main__":
    main()
