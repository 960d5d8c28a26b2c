"""Model-level smoke tests of the integrations, like the reference's (tests/test_models.py:6-38): a flash-linear-attention
layer and a one-layer Qwen3.5 model train one step with the optimized operators bound, the backward is counted, and
every gradient is finite."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(autouse=True)
def _restore():
    yield
    import rewy_b200 as fdr
    from rewy_b200 import integrations
    integrations.uninstall()
    fdr.disable()


def test_fla_delta_net_layer_uses_the_backend():
    pytest.importorskip("fla")
    import rewy_b200 as fdr
    from fla.layers.delta_net import DeltaNet          # imported before enable(), as a training script would
    torch.manual_seed(0)
    model = DeltaNet(hidden_size=256, num_heads=2, layer_idx=0).to(DEV).train()
    x = torch.randn(1, 128, 256, device=DEV, requires_grad=True)
    fdr.enable(ops=("delta",), integrations=("fla",))
    fdr.stats(reset=True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        out = model(x, use_cache=False)[0]
    out.float().square().mean().backward()
    fdr.assert_used(("delta",))
    assert torch.isfinite(x.grad).all()
    assert all(torch.isfinite(p.grad).all() for p in model.parameters() if p.grad is not None)
    assert not any("fallback" in k or "rejected" in k for k in fdr.stats())


def test_qwen3_5_adapter_trains_a_small_model():
    cfg_mod = pytest.importorskip("transformers.models.qwen3_5.configuration_qwen3_5")
    mdl_mod = pytest.importorskip("transformers.models.qwen3_5.modeling_qwen3_5")
    import rewy_b200 as fdr
    cfg = cfg_mod.Qwen3_5TextConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=1, num_attention_heads=2,
                                    num_key_value_heads=2, head_dim=128, vocab_size=256, linear_num_key_heads=2,
                                    linear_num_value_heads=2, linear_key_head_dim=128, linear_value_head_dim=128,
                                    layer_types=["linear_attention"], use_cache=False)
    cfg._attn_implementation = "sdpa"
    fdr.enable(ops=("gdn",), integrations=("qwen3_5",))     # before the model is built: layers bind at construction
    fdr.stats(reset=True)
    torch.manual_seed(0)
    model = mdl_mod.Qwen3_5ForCausalLM(cfg).to(DEV).train()
    tokens = torch.randint(0, 256, (1, 128), device=DEV)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        loss = model(input_ids=tokens, labels=tokens).loss
    loss.backward()
    fdr.assert_used(("gdn",))
    assert torch.isfinite(loss)
    assert all(torch.isfinite(p.grad).all() for p in model.parameters() if p.grad is not None)
    assert not any("fallback" in k or "rejected" in k for k in fdr.stats())
