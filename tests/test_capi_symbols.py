"""The C-ABI library loads without a GPU and exports every symbol include/b200moe.h declares (no compute calls here)."""
import re

from conftest import ROOT


def declared_symbols():
    text = (ROOT / "include" / "b200moe.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200moe_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound():
    import sm120fp4_b200._lib as L
    h = L.lib()
    names = declared_symbols()
    assert len(names) >= 19
    for n in names:
        assert hasattr(h, n), f"{n} declared in include/b200moe.h but not exported"
        assert n in L.SIGNATURES, f"{n} has no ctypes signature"
    assert sorted(L.SIGNATURES) == names
    assert h.b200moe_version() >= 100
    assert b"workspace" in h.b200moe_error_string(L.ERR_WORKSPACE)


def test_argument_errors_need_no_gpu():
    import sm120fp4_b200._lib as L
    h = L.lib()
    assert h.b200moe_to_128x4(None, None, 1, 1, 1, None) == L.ERR_ARG
    assert h.b200moe_quantize_nvfp4(None, 0, None, 1, 16, None, 0, None, None, 0, None) == L.ERR_ARG
    assert h.b200moe_route(None, 5, 8, 0, None, None, None, None, 0, None) == L.ERR_ARG
    assert h.b200moe_route_workspace_bytes(100, 8) > 0
    assert h.b200moe_layer_workspace_bytes(None) == L.ERR_ARG


def test_host_side_mirrors():
    import pytest
    import torch
    from sm120fp4_b200 import moe_layer, padded_sf_shape, vllm_backend as vb
    assert padded_sf_shape(100, 5) == (128, 8) and padded_sf_shape(1536, 128) == (1536, 128)
    # the selection rule states what runs (sm120fp4/kernels/moe_layer.py:60-93 is the reference's rule for its kernels)
    assert moe_layer.choice(1) == moe_layer.choice(16) == ("tcgen05_fused", "tcgen05_fused") and moe_layer.use_pdl(1) and moe_layer.use_pdl(16)
    assert moe_layer.choice(4, 2816, 704) == ("tcgen05_fused", "tcgen05_fused")            # the Gemma shape: no crossover below 16 tokens
    assert moe_layer.choice(4, 4096, 1024) == ("mma_sync_fused", "mma_sync_fused")          # x scale tiles no longer fit in TMEM
    assert moe_layer.regime(16) == "decode" and moe_layer.regime(17) == "decode_slices"
    assert moe_layer.regime(17, prefill=True) == "prefill_w4a4" and moe_layer.regime(4096, prefill=True, mid_max_tokens=256) == "prefill_w4a4"
    assert moe_layer.regime(32, mid_max_tokens=256, mid_min_tokens=33) == "decode_slices" and moe_layer.regime(33, mid_max_tokens=256) == "mid_w4a16"
    assert moe_layer.regime(257, mid_max_tokens=256) == "decode_slices" and moe_layer.regime(64, 4096, 1024, mid_max_tokens=256) == "decode_slices"
    assert moe_layer.regime(20, mid_max_tokens=128, mid_min_tokens=17) == "mid_w4a16"
    with pytest.raises(ValueError):
        moe_layer.choice(17)
    with pytest.raises(ValueError):
        moe_layer.choice(1, 2000, 768)
    k = vb.kernels()                                                                         # the reference's loader surface
    assert k.layer is moe_layer and callable(k.route.route) and callable(k.fc1_cc.fc1_w4a16) and callable(k.fc1_tc.fc1_mma)
    assert callable(k.fc2_cc.fc2_w4a16) and callable(k.fc2_pf.fc2_pf) and moe_layer.fc1.build() is k.fc1_cc
    vb.set_pdl(k, False)
    vb.set_pdl(k, True)
    t = torch.arange(24).reshape(2, 4, 3)
    assert torch.equal(vb.rotate_halves(vb.rotate_halves(t, 2), 2), t)
    assert torch.equal(vb.rotate_halves(t, 2)[:, :2], t[:, 2:])
    with pytest.raises(ValueError):   # unequal gate/up global scales (sm120fp4/vllm_backend.py:199-202)
        vb.weights_from_vllm_layout(torch.zeros(2, 128, 64, dtype=torch.uint8), torch.zeros(2, 128, 8, dtype=torch.uint8),
                                    torch.tensor([[1.0, 2.0], [1.0, 1.0]]), torch.zeros(2, 128, 32, dtype=torch.uint8),
                                    torch.zeros(2, 128, 4, dtype=torch.uint8), torch.ones(2), 2)
    with pytest.raises(TypeError):    # codes must be uint8 views
        vb.Weights(torch.zeros(2, 128, 64), torch.zeros(2, 128, 8, dtype=torch.uint8), torch.ones(2),
                   torch.zeros(2, 128, 32, dtype=torch.uint8), torch.zeros(2, 128, 4, dtype=torch.uint8), torch.ones(2), 2)
