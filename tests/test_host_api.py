"""Host-side mirror of the reference API: pieces that need no GPU."""
import types

import pytest
import torch
import torch.nn as nn

from dualquant_b200 import formats, quarot
from dualquant_b200.activations import PermLinear, install_perm_linear


def test_get_hadK_matches_reference_matrix(golden):
    had, k = quarot.get_hadK(14336)
    assert k == 28
    assert torch.equal(had, torch.from_numpy(golden["had28"]).float())
    assert quarot.get_hadK(4096) == (None, 1)
    h12, k12 = quarot.get_hadK(12 * 64)
    assert k12 == 12 and h12.shape == (12, 12)
    assert quarot.full_hadamard_scale(14336) == float((1.0 / torch.tensor(14336).sqrt()).item())


def test_make_format_surface():
    f = formats.make_format("rtn_int4", block_size=-1)
    assert (f.name, f.block_size, f.max_val) == ("rtn_int4", -1, 7.0)
    assert torch.equal(f.cast_element_only(torch.tensor([-9.4, 0.5, 1.5, 7.7])),
                       torch.tensor([-8.0, 0.0, 2.0, 7.0]))
    with pytest.raises(ValueError):
        formats.make_format("int3")
    with pytest.raises(RuntimeError):
        f.cast(torch.zeros(2, 128))  # CPU tensor: no CPU path


def test_perm_linear_attributes_and_install():
    parent = nn.Module()
    parent.down_proj = nn.Linear(256, 128, bias=False).to(torch.bfloat16)
    parent.o_proj = nn.Linear(256, 128, bias=False).to(torch.bfloat16)
    fmt = formats.make_format("rtn_int4", block_size=-1)
    pl = install_perm_linear(parent, "down_proj", fmt, col_scales=torch.ones(256, dtype=torch.float64))
    install_perm_linear(parent, "o_proj", fmt)
    assert isinstance(parent.down_proj, PermLinear) and parent.down_proj is pl
    assert pl.act_scale.dtype == torch.float32 and pl.dtype == torch.bfloat16
    for attr, val in (("online_full_had", False), ("online_partial_had", False), ("had_K", None),
                      ("K", 1), ("had_dim", 0), ("fp32_had", False), ("act_quant_enabled", True),
                      ("quantize_bmm_input", False)):
        assert getattr(pl, attr) == val if val is not None else getattr(pl, attr) is None
    pl.set_act_quant_enabled(0)
    assert pl.act_quant_enabled is False
    model = nn.Module()
    model.block = parent
    model.config = types.SimpleNamespace(intermediate_size=28 * 64, num_attention_heads=32,
                                         hidden_size=256, head_dim=None)
    quarot.install_online_hadamards(model)
    assert parent.down_proj.online_full_had and parent.down_proj.K == 28
    assert parent.o_proj.online_partial_had and parent.o_proj.K == 1 and parent.o_proj.had_dim == 8
    with pytest.raises(RuntimeError):
        pl(torch.zeros(2, 256, dtype=torch.bfloat16))  # CPU tensor


def test_hadamard_generators_reproduce_every_order_of_the_reference_table(golden):
    """quarot.hadamard_of_order builds each matrix of quarot/vendor/hadamard_utils.py:57-391 from its
    construction (Paley I / II, Sylvester doubling, Williamson); the fixture holds the reference's
    own literals, one bit per entry."""
    import numpy as np
    import torch

    from dualquant_b200 import quarot

    bits, off = golden["had_bits"], 0
    for k in golden["had_orders"].tolist():
        nbytes = (k * k + 7) // 8
        ref = np.unpackbits(bits[off:off + nbytes])[: k * k].reshape(k, k).astype(np.float32) * 2 - 1
        off += nbytes
        h = quarot.hadamard_of_order(k)
        assert torch.equal(h, torch.from_numpy(ref)), k
        assert torch.equal(h @ h.T, k * torch.eye(k))
    # the decomposition get_hadK picks (first matching order of the reference's list)
    for n, k in ((11008, 172), (14336, 28), (13824, 108), (6656, 52), (4096, 1), (15360, 60), (17920, 140),
                 (1280, 40), (1536, 12), (1152, 36), (4992, 156)):
        h, kk = quarot.get_hadK(n)
        assert kk == k and (h is None) == (k == 1)
    ht, _ = quarot.get_hadK(11008, transpose=True)
    assert torch.equal(ht, quarot.hadamard_of_order(172).T)


def test_column_scale_files_load_and_install(tmp_path, golden):
    """wrap.load_column_scales / install_column_scales on a file with the layout of the reference's
    shipped scale files (key names and widths of one of them are in the golden fixture)."""
    import torch
    import torch.nn as nn

    from dualquant_b200 import formats, wrap
    from dualquant_b200.activations import PermLinear

    keys = [str(k) for k in golden["beta_file_keys"]]
    widths = golden["beta_file_widths"].tolist()
    assert "layer0.mlp.down_proj" in keys and int(golden["beta_file_count"][0]) % 7 == 0
    blob = {k: torch.rand(w) + 0.5 for k, w in zip(keys, widths)}
    path = tmp_path / "scales.pt"
    torch.save(blob, path)
    scales = wrap.load_column_scales(str(path))
    assert sorted(scales) == sorted(keys) and all(v.dtype == torch.float32 for v in scales.values())

    fmt = formats.make_format("rtn_int4", block_size=-1)

    def block(idx):
        layer = nn.Module()
        for k, w in zip(keys, widths):
            head, _, p = k.partition(".")
            if head != f"layer{idx}":
                continue
            parent_name, leaf = p.split(".")
            if not hasattr(layer, parent_name):
                setattr(layer, parent_name, nn.Module())
            setattr(getattr(layer, parent_name), leaf, PermLinear(nn.Linear(w, 8, bias=False), fmt))
        return layer

    n_layers = 1 + max(int(k.split(".")[0][5:]) for k in keys)
    model = nn.Module()
    model.model = nn.Module()
    model.model.layers = nn.ModuleList([block(i) for i in range(n_layers)])
    assert wrap.install_column_scales(model, scales) == len(keys)
    got = model.model.layers[0].mlp.down_proj.act_scale
    assert torch.equal(got, blob["layer0.mlp.down_proj"])
    torch.save({"oops": torch.ones(3)}, path)
    with pytest.raises(ValueError):
        wrap.load_column_scales(str(path))


def test_status_word_decoding():
    """dq_device_status packs DQ_ERR_TIMEOUT with the site code in the upper 16 bits; the binding
    raises RuntimeError for it (not ValueError: it is not an argument error)."""
    from dualquant_b200 import _lib

    with pytest.raises(RuntimeError, match="DQ_ERR_TIMEOUT"):
        _lib.check(_lib.DQ_ERR_TIMEOUT | (23 << 16), "dq_device_status")
    with pytest.raises(ValueError, match="DQ_ERR_SHAPE"):
        _lib.check(1, "dq_x")
    _lib.check(0, "dq_x")
