"""The vLLM-facing classes (sm120fp4/vllm_classes.py in the reference): `fits`, the checkpoint-layout loader
(`process_weights_after_loading` on a stand-in layer filled the way vLLM's weight loader fills it) and `apply`.
vLLM itself is only imported, never started."""
from types import SimpleNamespace as NS

import numpy as np
import pytest
import torch

vc = pytest.importorskip("sm120fp4_b200.vllm_classes", reason="vLLM is not importable here")
from vllm.model_executor.layers.fused_moe.activation import MoEActivation  # noqa: E402


def moe_config(**kw):
    base = dict(is_act_and_mul=True, activation=MoEActivation.SILU, hidden_dim=2048, intermediate_size_per_partition=768,
                moe_parallel_config=NS(use_ep=False), in_dtype=torch.bfloat16)
    base.update(kw)
    return NS(**base)


def test_fits_accepts_the_reference_shapes_and_more():
    fits = vc.SM120Fp4MoEMethod.fits
    assert fits(moe_config()) == (True, "")
    assert fits(moe_config(intermediate_size_per_partition=1024))[0]
    assert fits(moe_config(hidden_dim=2816, intermediate_size_per_partition=704))[0]      # the Gemma-4 shape
    assert fits(moe_config(moe_parallel_config=NS(use_ep=True), num_local_experts=16))[0]  # expert parallelism is taken


@pytest.mark.parametrize("kw,word", [
    (dict(activation=MoEActivation.GELU), "SiLU"), (dict(is_act_and_mul=False), "SiLU"),
    (dict(hidden_dim=2000), "hidden size"), (dict(intermediate_size_per_partition=700), "intermediate size"),
    (dict(in_dtype=torch.float16), "bf16"), (dict(num_local_experts=512), "at most 256"), (dict(experts_per_token=32), "at most 16")])
def test_fits_declines_with_a_reason(kw, word):
    ok, why = vc.SM120Fp4MoEMethod.fits(moe_config(**kw))
    assert not ok and word in why


def test_class_name_keeps_modelopt_and_alias():
    assert "ModelOpt" in vc.ModelOptNvFp4FusedMoESM120.__name__       # vLLM's weight loader branches on the class name
    assert vc.SM120Fp4MoEMethod is vc.ModelOptNvFp4FusedMoESM120
    from sm120fp4_b200 import vllm_backend as vb
    ns = vb.classes()
    assert ns.Config is vc.SM120Fp4Config and ns.Method is vc.SM120Fp4MoEMethod


def test_apply_refuses_what_the_kernels_do_not_do():
    m = object.__new__(vc.SM120Fp4MoEMethod)
    m.weights = NS(forward=lambda *a: pytest.fail("must not run"))
    x = torch.zeros(1, 128, dtype=torch.bfloat16)
    with pytest.raises(NotImplementedError, match="shared experts"):
        m.apply(NS(), x, None, None, object(), None)
    with pytest.raises(NotImplementedError, match="apply_router_weight_on_input"):
        m.apply(NS(apply_router_weight_on_input=True), x, None, None, None, None)


def test_expert_map_masks_other_ranks_experts():
    """With an expert map the local shard runs with the other ranks' slots masked (id -1, weight 0): partial rows."""
    from sm120fp4_b200.vllm_backend import map_expert_ids
    emap = torch.tensor([-1, -1, -1, -1, 0, 1, 2, 3])                    # this rank owns global experts 4..7
    ids = torch.tensor([[0, 5], [7, 4], [2, 3]], dtype=torch.int32)
    wts = torch.tensor([[0.25, 0.75], [0.5, 0.5], [0.9, 0.1]])
    lid, lw = map_expert_ids(ids, wts, emap)
    assert lid.tolist() == [[-1, 1], [3, 0], [-1, -1]] and lid.dtype == torch.int32
    assert lw.tolist() == [[0.0, 0.75], [0.5, 0.5], [0.0, 0.0]]
    seen = {}
    m = object.__new__(vc.SM120Fp4MoEMethod)
    m.weights = NS(forward=lambda x, i, w: seen.update(ids=i, wts=w) or x)
    m.apply(NS(expert_map=emap), torch.zeros(3, 128, dtype=torch.bfloat16), wts, ids, None, None)
    assert seen["ids"].tolist() == lid.tolist() and seen["wts"].tolist() == lw.tolist()


def test_register_is_a_no_op_without_the_switch(monkeypatch):
    from sm120fp4_b200 import vllm_backend as vb
    monkeypatch.delenv(vb.ENV, raising=False)
    assert vb.register() is False


# ------------------------------------------------------------------------------------------------------------------ GPU
class CheckpointLayer(torch.nn.Module):
    """What vLLM's loader leaves on a routed-experts layer of a ModelOpt NVFP4 checkpoint: w13 as [gate; up]."""

    def __init__(self, q1_up_gate, s1_up_gate, a1, q2, s2, a2, top_k, input_scales=True):
        super().__init__()
        inter = q1_up_gate.shape[1] // 2
        back = lambda t: torch.cat([t[:, inter:], t[:, :inter]], dim=1).contiguous()      # [up; gate] -> [gate; up]
        P = lambda t: torch.nn.Parameter(t, requires_grad=False)
        self.w13_weight, self.w13_weight_scale = P(back(q1_up_gate)), P(back(s1_up_gate).view(torch.float8_e4m3fn))
        self.w13_weight_scale_2 = P(torch.stack([a1, a1], dim=1))
        self.w2_weight, self.w2_weight_scale, self.w2_weight_scale_2 = P(q2), P(s2.view(torch.float8_e4m3fn)), P(a2)
        if input_scales:
            e = q2.shape[0]
            self.w13_input_scale = P(torch.ones(e, 2, device=q2.device))
            self.w2_input_scale = P(torch.ones(e, device=q2.device))
        self.top_k = top_k


def _method():
    m = object.__new__(vc.SM120Fp4MoEMethod)      # without vLLM's FusedMoEConfig: only the loader and apply are under test
    m.weights = None
    return m


@pytest.mark.gpu
@pytest.mark.parametrize("tokens", [1, 5, 16, 40])
def test_loader_and_apply_match_the_oracle(tokens):
    import sm120fp4_b200 as pkg
    from helpers import check_layer_output, check_w4a4_output
    from oracle import nvfp4_oracle as O
    from sm120fp4_b200 import synth
    e, h, i, k = 8, 256, 128, 2
    w13, w2 = synth.layer_weights_bf16(e, h, i, seed=3)
    q1, s1, g1 = pkg.quantize_nvfp4_experts(w13.cuda())
    q2, s2, g2 = pkg.quantize_nvfp4_experts(w2.cuda())
    a1, a2 = 1.0 / g1, 1.0 / g2
    layer = CheckpointLayer(q1, s1, a1, q2, s2, a2, k)
    m = _method()
    m.process_weights_after_loading(layer)
    assert layer.w13_input_scale is None and layer.w2_input_scale is None         # consumed, as in the reference
    assert torch.equal(layer.w13_weight.data, q1)                                  # stored [up; gate], the kernels' order
    assert m.weights.prefill is not None
    g = torch.Generator().manual_seed(tokens)
    x = (torch.randn(tokens, h, generator=g) * 0.5).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(tokens)]).to(torch.int32)
    wts = torch.softmax(torch.randn(tokens, k, generator=g), dim=-1)
    out = m.apply(layer, x.cuda(), wts.cuda(), ids.cuda(), None, None)
    m.weights.status()
    ow = O.ExpertWeights(q1.cpu().numpy(), s1.cpu().numpy(), a1.cpu().numpy(), q2.cpu().numpy(), s2.cpu().numpy(), a2.cpu().numpy())
    want = O.moe_reference(x.float().numpy(), ow, ids.numpy(), wts.numpy(), act_quant=tokens > 16)
    (check_w4a4_output if tokens > 16 else check_layer_output)(out, want, f"vllm method, {tokens} tokens")


@pytest.mark.gpu
def test_loader_refuses_unequal_gate_and_up_scales_and_runs_slices_without_input_scales():
    import sm120fp4_b200 as pkg
    from sm120fp4_b200 import synth
    e, h, i, k = 4, 128, 64, 2
    w13, w2 = synth.layer_weights_bf16(e, h, i, seed=4)
    q1, s1, g1 = pkg.quantize_nvfp4_experts(w13.cuda())
    q2, s2, g2 = pkg.quantize_nvfp4_experts(w2.cuda())
    layer = CheckpointLayer(q1, s1, 1.0 / g1, q2, s2, 1.0 / g2, k, input_scales=False)
    m = _method()
    m.process_weights_after_loading(layer)
    assert m.weights.prefill is None
    out = m.apply(layer, torch.zeros(20, h, dtype=torch.bfloat16, device="cuda"), torch.ones(20, k, device="cuda") / k,
                  torch.zeros(20, k, dtype=torch.int32, device="cuda") + torch.arange(k, device="cuda", dtype=torch.int32), None, None)
    assert out.shape == (20, h) and float(out.float().abs().max()) == 0.0
    bad = CheckpointLayer(q1, s1, 1.0 / g1, q2, s2, 1.0 / g2, k)
    bad.w13_weight_scale_2.data[1, 1] *= 2
    with pytest.raises(ValueError, match="gate and up global scales differ on 1 of 4"):
        _method().process_weights_after_loading(bad)
