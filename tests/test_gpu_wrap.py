"""DualQuant offline outputs (mat_q, column scales) -> packed artefact -> PermLinear."""
import os
import sys

import pytest
import torch
import torch.nn as nn

sys.path.insert(0, os.path.join(os.path.dirname(__file__), ".."))

from oracle import dq_oracle as oracle  # noqa: E402


def _exact_fake_quant(N, K, seed):
    """Codes and fp16 group scales whose product is exactly representable in bf16, with a +-7 in
    every group so that re-quantising the product must return the same codes and scales."""
    g = torch.Generator().manual_seed(seed)
    codes = torch.randint(-7, 8, (N, K), generator=g, dtype=torch.int8)
    codes.view(N, K // 128, 128)[:, :, 0] = 7
    mant = torch.randint(0, 4, (N, K // 128), generator=g).float()
    expo = torch.randint(-9, -5, (N, K // 128), generator=g).float()
    sw = ((1.0 + mant / 4.0) * torch.exp2(expo)).half()
    mat_q = (codes.float().view(N, K // 128, 128) * sw.float()[:, :, None]).view(N, K)
    assert torch.equal(mat_q.bfloat16().float(), mat_q)
    return codes, sw, mat_q.bfloat16()


def test_load_wrap_cache_roundtrip(tmp_path):
    from dualquant_b200 import wrap
    blob = {"mat_q": torch.randn(8, 128), "beta": torch.rand(128) + 0.5}
    path = tmp_path / "layer.pt"
    torch.save(blob, path)
    got = wrap.load_wrap_cache(str(path))
    assert torch.equal(got["mat_q"], blob["mat_q"]) and torch.equal(got["beta"], blob["beta"])
    torch.save({"weights": 1}, path)
    with pytest.raises(ValueError):
        wrap.load_wrap_cache(str(path))


@pytest.mark.gpu
def test_pack_from_dualquant_recovers_codes_exactly():
    from dualquant_b200 import ops, wrap
    dev = torch.device("cuda", 0)
    N, K = 384, 1024
    codes, sw, mat_q = _exact_fake_quant(N, K, 3)
    beta = torch.rand(K) + 0.5
    pw, a = wrap.pack_from_dualquant(mat_q.to(dev), beta)
    assert torch.equal(ops.unpack_w_int4(pw).cpu(), codes)
    # sw_t is [row tile][group][128 rows]
    got_sw = pw.sw_t.view(N // 128, K // 128, 128).permute(0, 2, 1).reshape(N, K // 128)
    assert torch.equal(got_sw.cpu(), sw)
    assert torch.equal(a.cpu(), beta.float())


@pytest.mark.gpu
def test_install_from_wrap_matches_oracle():
    from dualquant_b200 import formats, wrap
    dev = torch.device("cuda", 0)
    N, K, M = 256, 512, 24
    codes, sw, mat_q = _exact_fake_quant(N, K, 5)
    beta = torch.exp(torch.randn(K, generator=torch.Generator().manual_seed(1)) * 0.3)
    parent = nn.Module()
    parent.proj = nn.Linear(K, N, bias=False).to(dev).bfloat16()
    perm = wrap.install_from_wrap(parent, "proj", mat_q, beta, formats.make_format("rtn_int4", block_size=-1))
    assert parent.proj is perm and perm._packed is not None
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(2)).bfloat16()
    y = perm(x.to(dev)).float().cpu()
    qx, sx = oracle.quant_act_int4(x, beta.float(), scale_fp16=False)[:2]
    ref = oracle.epilogue(oracle.acc_int32(qx, codes), sw, None, sx)
    err = (y - ref).abs().max() / ref.abs().max()
    assert err < 8e-3, err  # bf16 output rounding of the module
