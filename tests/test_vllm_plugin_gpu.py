"""Converter -> checkpoint tensors -> vLLM linear method -> output, on one GPU."""
import pytest
import torch

from tests import helpers as H

pytestmark = pytest.mark.gpu


def test_converted_checkpoint_runs_through_the_plugin():
    pytest.importorskip("vllm", reason="vLLM is not installed")
    try:
        from sharq_b200 import vllm_plugin as plugin
    except Exception as exc:
        pytest.skip(f"vLLM could not be imported: {exc}")
    from sharq_b200 import checkpoint as C
    from sharq_b200 import ops

    h, f, heads_q, heads_kv, d = 512, 1024, 4, 2, 128
    state = {}
    p = "model.layers.0"
    for name, (n, k) in {"self_attn.q_proj": (heads_q * d, h), "self_attn.k_proj": (heads_kv * d, h),
                         "self_attn.v_proj": (heads_kv * d, h), "self_attn.o_proj": (h, heads_q * d),
                         "mlp.gate_proj": (f, h), "mlp.up_proj": (f, h), "mlp.down_proj": (h, f)}.items():
        state[f"{p}.{name}.weight"] = H.config0_w(n, k, len(name))
    state[f"{p}.self_attn.q_proj.bias"] = torch.zeros(heads_q * d, dtype=torch.bfloat16)
    state[f"{p}.self_attn.k_proj.bias"] = torch.ones(heads_kv * d, dtype=torch.bfloat16)
    state[f"{p}.self_attn.v_proj.bias"] = torch.zeros(heads_kv * d, dtype=torch.bfloat16)
    state["model.norm.weight"] = torch.ones(h, dtype=torch.bfloat16)
    ckpt = C.convert_state_dict(state, 1)
    assert f"{p}.self_attn.qkv_proj.QW" in ckpt and f"{p}.mlp.gate_up_proj.SFW_dense" in ckpt
    assert f"{p}.self_attn.q_proj.weight" not in ckpt and "model.norm.weight" in ckpt
    assert ckpt[f"{p}.self_attn.qkv_proj.bias"].numel() == (heads_q + 2 * heads_kv) * d

    base = f"{p}.mlp.gate_up_proj"
    entry = C.layer_entry(ckpt, base)
    method = plugin.SHARQLinearMethod(plugin.SHARQConfig(), prefix=base)
    layer = torch.nn.Module()
    method.create_weights(layer, h, [f, f], h, 2 * f, torch.bfloat16)
    for name in ("QW", "SFW_sparse", "SFW_dense", "scale_b"):
        getattr(layer, name).weight_loader(getattr(layer, name), entry[name])
    x = H.config0_x(96, h, 1).cuda().view(2, 48, h)
    got = method.apply(layer, x)
    want = ops.sharq_linear_forward(x.view(-1, h), entry["QW"].cuda(), entry["SFW_sparse"].cuda(), entry["SFW_dense"].cuda(),
                                    float(entry["scale_b"].item()))
    ops.check_device_errors()
    assert got.shape == (2, 48, 2 * f)
    assert torch.equal(got.view(-1, 2 * f), want)
    # and against the unquantised product, loosely (W4A4)
    ref = x.view(-1, h).float() @ torch.cat((state[f"{p}.mlp.gate_proj.weight"], state[f"{p}.mlp.up_proj.weight"])).float().cuda().T
    rel = (got.view(-1, 2 * f).float() - ref).norm() / ref.norm()
    assert rel < 0.2, float(rel)
