"""Generates tests/golden/*.npz by running the REFERENCE's own Python code on CPU.

Run in the authoring container only (it needs the reference checkout):

    python tests/golden/make_golden.py <path of the reference checkout>

The fixtures are small seeded input/output pairs of the reference functions on the W4A4 hot
path; tests compare the oracle (oracle/dq_oracle.py) and the CUDA library against them.  The
reference is imported through three shims, none of which touches the arithmetic recorded here:
  * BLOCKFMT_BACKEND -> an in-memory stub module exposing `Format` (the reference imports
    blockfmt at module import time even for rtn_int4; the external package's own MX/NVFP4 casts
    are NOT recorded - the MXFP4 fixture comes from the reference's in-tree convert_to_mxfp);
  * stub `accelerate` modules (imported, never called, by quarot/vendor/utils.py);
  * the reference's own pure-torch stand-in for fast_hadamard_transform.
"""
from __future__ import annotations

import os
import sys
import types

import numpy as np
import torch


def _install_shims(ref_root: str) -> None:
    stub = types.ModuleType("_dq_blockfmt_stub")

    class Format:  # never exercised by the fixtures
        @classmethod
        def from_shorthand(cls, s):
            return cls()

        def cast(self, t, axis=-1):
            raise RuntimeError("blockfmt stub: block casts are not part of the golden fixtures")

    stub.Format = Format
    sys.modules["_dq_blockfmt_stub"] = stub
    os.environ["BLOCKFMT_BACKEND"] = "_dq_blockfmt_stub"
    import transformers  # noqa: F401  (must precede the accelerate stubs)

    acc = types.ModuleType("accelerate")
    acc_utils = types.ModuleType("accelerate.utils")
    for name in ("dispatch_model", "infer_auto_device_map"):
        setattr(acc, name, lambda *a, **k: None)
    acc_utils.get_balanced_memory = lambda *a, **k: None
    acc.utils = acc_utils
    sys.modules.setdefault("accelerate", acc)
    sys.modules.setdefault("accelerate.utils", acc_utils)
    sys.path.insert(0, ref_root)
    sys.path.insert(0, os.path.join(ref_root, "vendor", "dualscale_kernel_benchmark"))


def _seeded_x(M, K, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g)
    out_ch = torch.randperm(K, generator=g)[: max(1, K // 100)]
    x[:, out_ch] *= 20
    return x.to(torch.bfloat16)


def main(ref_root: str) -> None:
    _install_shims(ref_root)
    import torch.nn as nn
    from activations.perm_linear import PermLinear  # reference
    from formats import make_format  # reference
    import hadamard_utils  # reference (vendored QuaRot)
    from torch_quant import float_to_fp4  # reference

    here = os.path.dirname(os.path.abspath(__file__))
    out = {}

    # ---- Hadamard matrix and decomposition --------------------------------------------------
    had28, k28 = hadamard_utils.get_hadK(14336)
    assert k28 == 28
    out["had28"] = had28.numpy().astype(np.int8)
    _, k1 = hadamard_utils.get_hadK(32)
    assert k1 == 1
    # every order of the reference's table (quarot/vendor/hadamard_utils.py:5-55), one bit per entry
    orders = (12, 20, 28, 36, 40, 52, 60, 108, 140, 156, 172)
    out["had_orders"] = np.array(orders, dtype=np.int32)
    out["had_bits"] = np.concatenate([
        np.packbits((getattr(hadamard_utils, f"get_had{k}")().numpy() > 0).reshape(-1)) for k in orders])

    # ---- per-token rtn_int4 cast (formats/rtn_int.py) ---------------------------------------
    fmt = make_format("rtn_int4", block_size=-1)
    g = torch.Generator().manual_seed(1)
    x = _seeded_x(24, 512, 11)
    a = torch.exp(torch.randn(512, generator=g) * 0.3).to(torch.float16).to(torch.float32)
    x32 = x.float() * a
    x32[5] = 0.0  # all-zero token
    out["cast_in"] = x32.numpy()
    out["cast_out"] = fmt.cast(x32).numpy()

    # ---- weight cast with groups of 128 -------------------------------------------------------
    wfmt = make_format("rtn_int4", block_size=128)
    w = (torch.randn(64, 512, generator=g) * 0.02).to(torch.bfloat16).float()
    out["wcast_in"] = w.numpy()
    out["wcast_out"] = wfmt.cast(w).numpy()

    # ---- PermLinear forward: plain, full Hadamard (28 x 32), partial Hadamard -----------------
    def run_perm(K, N, M, seed, mode):
        gg = torch.Generator().manual_seed(seed)
        lin = nn.Linear(K, N, bias=False).to(torch.bfloat16)
        wq = wfmt.cast((torch.randn(N, K, generator=gg) * 0.02).to(torch.bfloat16).float())
        lin.weight.data = wq.to(torch.bfloat16)
        pl = PermLinear(lin, fmt)
        aa = torch.exp(torch.randn(K, generator=gg) * 0.3).to(torch.float16).to(torch.float32)
        pl.set_act_scale(aa)
        if mode == "full":
            pl.online_full_had = True
            pl.had_K, pl.K = hadamard_utils.get_hadK(K)
        elif mode == "partial":
            pl.online_partial_had = True
            pl.had_K, pl.K = hadamard_utils.get_hadK(K // 8)
            pl.had_dim = 8
        xx = _seeded_x(M, K, seed + 100)
        with torch.no_grad():
            xq = pl._quantise_act(xx)
            y = pl(xx)
        return {
            "x": xx.view(torch.int16).numpy(),  # bf16 bit patterns
            "a": aa.numpy(),
            "w_bf16": lin.weight.data.view(torch.int16).numpy(),
            "xq_bf16": xq.view(torch.int16).numpy(),
            "y_bf16": y.view(torch.int16).numpy(),
        }

    # PermLinear with neither activation scale nor Hadamard: the bf16-arithmetic branch
    gg = torch.Generator().manual_seed(31)
    lin0 = nn.Linear(512, 128, bias=False).to(torch.bfloat16)
    lin0.weight.data = wfmt.cast((torch.randn(128, 512, generator=gg) * 0.02).to(torch.bfloat16).float()).to(torch.bfloat16)
    pl0 = PermLinear(lin0, fmt)
    x0 = _seeded_x(24, 512, 131)
    x0[3] = 0
    with torch.no_grad():
        out["perm_noscale_x"] = x0.view(torch.int16).numpy()
        out["perm_noscale_w_bf16"] = lin0.weight.data.view(torch.int16).numpy()
        out["perm_noscale_xq_bf16"] = pl0._quantise_act(x0).view(torch.int16).numpy()
        out["perm_noscale_y_bf16"] = pl0(x0).view(torch.int16).numpy()

    for tag, (K, N, M, mode) in {
        "plain": (512, 128, 20, "none"),
        "full": (896, 128, 12, "full"),  # 896 = 28 * 32
        "partial": (256, 128, 12, "partial"),  # 32 heads x head_dim 8
    }.items():
        for k, v in run_perm(K, N, M, 7, mode).items():
            out[f"perm_{tag}_{k}"] = v

    # ---- Hadamard alone (fp32) ------------------------------------------------------------------
    xh = torch.randn(6, 896, generator=g)
    hk, kk = hadamard_utils.get_hadK(896)
    out["hadfull_in"] = xh.numpy()
    out["hadfull_out"] = hadamard_utils.matmul_hadU_cuda(xh.clone(), hk, kk).numpy()

    # ---- reference packing / dequant (vendor kernel directory) ---------------------------------
    import fused_dual_scale_kernel as fdk  # needs triton importable; no GPU used here

    wp = torch.randn(32, 256, generator=g)
    packed, scale1 = fdk.pack_int4_weights(wp, 128)
    out["refpack_w"] = wp.numpy()
    out["refpack_packed"] = packed.numpy()
    out["refpack_scale_bf16"] = scale1.view(torch.int16).numpy()
    out["refpack_dequant"] = fdk.dequant_int4_reference(packed, scale1, 128).numpy()

    # ---- FP4 element rounding ---------------------------------------------------------------------
    grid = torch.cat([torch.linspace(-7, 7, 449), torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])])
    out["fp4_in"] = grid.numpy()
    out["fp4_out"] = float_to_fp4(grid.clone()).numpy()

    # ---- MXFP4 block cast: the reference's in-tree statement (legacy_vendor/torch_quant.py:359-375)
    # convert_to_mxfp moves its input to 'cuda:0'; there is no GPU where this script runs, so the
    # device argument is dropped for the duration of the call (the arithmetic is untouched).
    from torch_quant import convert_to_mxfp  # reference

    xm = _seeded_x(16, 512, 23).float()
    am = torch.exp(torch.randn(512, generator=g) * 0.3).to(torch.float16).to(torch.float32)
    xm = xm * am
    xm[3, 64:96] = 0.0            # an all-zero block
    xm[4, :] *= 2.0 ** -20        # small magnitudes
    xm[5, :] *= 2.0 ** 30         # large magnitudes
    xm[6, 0:32] = torch.tensor([6.0, -6.0, 3.0, 1.5] * 8)  # block maximum exactly on the grid
    xm[7, 0:32] = torch.tensor([4.0, 2.5, 1.25, 0.25] * 8) * 0.5  # elements on rounding ties
    orig_to = torch.Tensor.to

    def _to_without_cuda(self, *args, **kwargs):
        args = tuple(v for v in args if not (isinstance(v, str) and v.startswith("cuda")))
        kwargs = {k: v for k, v in kwargs.items() if not (k == "device" and str(v).startswith("cuda"))}
        return orig_to(self, *args, **kwargs) if (args or kwargs) else self

    torch.Tensor.to = _to_without_cuda
    try:
        out["mxfp4_in"] = xm.numpy().copy()
        out["mxfp4_out"] = convert_to_mxfp(xm.clone(), block_size=32).numpy()
    finally:
        torch.Tensor.to = orig_to

    # ---- E4M3 scale quantiser used for NVFP4-style block scales (scale_formats.py:39-45) -----------
    import scale_formats  # reference

    sgrid = torch.cat([torch.tensor([0.0, 1e-9, 2.0 ** -10, 2.0 ** -7, 2.0 ** -6, 0.0165, 447.0, 448.0, 449.0,
                                     500.0, 1e6]),
                       torch.exp(torch.linspace(-8.0, 7.0, 600))])
    out["e4m3_scale_in"] = sgrid.numpy()
    out["e4m3_scale_out"] = scale_formats.quantize_scale_e4m3(sgrid.clone()).numpy()

    # ---- QuaRot offline folds (quarot/llama_quarot.py:186-264) on a tiny random Llama ---------------
    # The reference moves weights with .cuda() inside apply_exact_had_to_linear; there is no GPU where
    # this script runs, so Tensor.cuda is the identity for the duration of the call.
    import transformers
    from quarot import llama_quarot

    tiny = transformers.LlamaConfig(hidden_size=64, intermediate_size=112, num_hidden_layers=1,
                                    num_attention_heads=4, num_key_value_heads=4, vocab_size=48,
                                    max_position_embeddings=32, tie_word_embeddings=False)
    torch.manual_seed(77)
    hf = transformers.LlamaForCausalLM(tiny).to(torch.float32)
    for prm in hf.parameters():  # norms away from 1 so that the fusion is visible
        if prm.dim() == 1:
            prm.data = torch.rand_like(prm) + 0.5
    names = ["model.embed_tokens.weight", "lm_head.weight", "model.norm.weight",
             "model.layers.0.input_layernorm.weight", "model.layers.0.post_attention_layernorm.weight"] + [
        f"model.layers.0.self_attn.{n}_proj.weight" for n in "qkvo"] + [
        f"model.layers.0.mlp.{n}_proj.weight" for n in ("gate", "up", "down")]
    sd = hf.state_dict()
    for nme in names:
        out["r1_before__" + nme] = sd[nme].numpy().copy()
    orig_cuda = torch.Tensor.cuda
    torch.Tensor.cuda = lambda self, *a, **k: self
    try:
        torch.manual_seed(78)  # random_hadamard_matrix draws its +-1 diagonal from the global generator
        llama_quarot.apply_r1(hf, rotate_mode="hadamard", apply_r2_r4=True)
    finally:
        torch.Tensor.cuda = orig_cuda
    sd = hf.state_dict()
    for nme in names:
        if nme in sd:
            out["r1_after__" + nme] = sd[nme].numpy().copy()

    # ---- format of the shipped column-scale files (scales_dualquant_rtn_int4/*.pt) -----------------
    scale_file = os.path.join(ref_root, "scales_dualquant_rtn_int4",
                              "DQ_Qwen_Qwen3-0.6B_iter15_scale_row_column_row_all_one_col_l1_norm_rtn_int4.pt")
    blob = torch.load(scale_file, map_location="cpu")
    keys = sorted(blob.keys())
    out["beta_file_keys"] = np.array(keys[:14])
    out["beta_file_count"] = np.array([len(keys)], dtype=np.int32)
    out["beta_file_widths"] = np.array([blob[k].numel() for k in keys[:14]], dtype=np.int32)
    out["beta_file_sample"] = blob["layer0.mlp.down_proj"][:32].numpy()

    # ---- DualQuant block-coordinate descent (layer_wrapper_dualquant.wrap_dualquant_layer) ----------
    # rtn_int4, element-mode inner quantiser, act_quant_flag=True: the layer keeps mat_q, the call
    # returns the column scales.  Configurations: 15 iterations of row_column with unrounded row
    # scales (rows max_abs, columns l1_norm), a max_abs / l2_norm one with E4M3 row scales, an E8M0
    # one, and column-only scales.  (The row_init="all_one" + col_init="l1_norm" combination in the
    # name of the shipped scale files drives every code of this synthetic matrix to zero in the
    # first step and the reference returns NaN; it is not recorded.)
    from layer_wrapper_dualquant import wrap_dualquant_layer

    g = torch.Generator().manual_seed(99)
    wb = torch.randn(96, 256, generator=g) * 0.02
    wb[:, torch.randperm(256, generator=g)[:4]] *= 12.0
    out["bcd_w"] = wb.numpy().copy()
    bcd_cfgs = {
        "iter15": dict(scale_option="row_column", row_init="max_abs", col_init="l1_norm", num_iter=15, scale_format="none"),
        "e4m3": dict(scale_option="row_column", row_init="max_abs", col_init="l2_norm", num_iter=5, scale_format="e4m3"),
        "e8m0": dict(scale_option="row_column", row_init="max_abs", col_init="l1_norm", num_iter=5, scale_format="e8m0"),
        "colonly": dict(scale_option="only_column", row_init="max_abs", col_init="l1_norm", num_iter=5, scale_format="none"),
    }
    for tag, c in bcd_cfgs.items():
        lin = torch.nn.Linear(256, 96, bias=False)
        lin.weight.data.copy_(wb)
        cfg = dict(num_splits=1, block_size=128, dualquant_to_element_tensor=True, **c)
        cs = wrap_dualquant_layer(lin, None, cfg, "rtn_int4", act_quant_flag=True)
        out[f"bcd_{tag}_matq"] = lin.weight.data.numpy().copy()
        out[f"bcd_{tag}_colscales"] = cs.numpy().copy()

    path = os.path.join(here, "reference_vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <path of the reference checkout>")
    main(sys.argv[1])
