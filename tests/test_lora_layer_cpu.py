"""LoRA layer: residual and relu^2 options of the fused forward, values and gradients against autograd on the statement."""
import pytest
import torch

from rwkvtune_b200.peft.lora.layer import LoraLinear


@pytest.mark.parametrize("mode", ["plain", "residual", "relu_sq"])
def test_lora_linear_options_match_the_plain_statement(mode):
    torch.manual_seed(3)
    base = torch.nn.Linear(24, 40, bias=False)
    base.weight.requires_grad_(False)
    layer = LoraLinear(base, r=8, lora_alpha=16)
    with torch.no_grad():
        layer.lora_B.normal_(0, 0.1)
    x = torch.randn(5, 7, 24, requires_grad=True)
    res = torch.randn(5, 7, 40, requires_grad=True) if mode == "residual" else None
    y = layer(x, residual=res, act="relu_sq" if mode == "relu_sq" else None)
    dy = torch.randn_like(y)
    y.backward(dy)
    got = [x.grad.clone(), layer.lora_A.grad.clone(), layer.lora_B.grad.clone()] + ([res.grad.clone()] if res is not None else [])

    x2 = x.detach().clone().requires_grad_(True)
    A = layer.lora_A.detach().clone().requires_grad_(True)
    B = layer.lora_B.detach().clone().requires_grad_(True)
    r2 = res.detach().clone().requires_grad_(True) if res is not None else None
    pre = x2 @ base.weight.t() + layer.scaling * (x2 @ A.t()) @ B.t()
    want_y = torch.relu(pre) ** 2 if mode == "relu_sq" else (pre + r2 if r2 is not None else pre)
    want_y.backward(dy)
    want = [x2.grad, A.grad, B.grad] + ([r2.grad] if r2 is not None else [])
    assert torch.allclose(y, want_y, atol=1e-5, rtol=1e-5)
    for g, w in zip(got, want):
        assert torch.allclose(g, w, atol=1e-4, rtol=1e-4)


def test_lora_linear_refuses_activation_with_residual():
    layer = LoraLinear(torch.nn.Linear(8, 8, bias=False), r=4)
    with pytest.raises(ValueError):
        layer(torch.randn(2, 8), residual=torch.randn(2, 8), act="relu_sq")


def test_merged_and_disabled_adapters_apply_the_options_after_the_base_layer():
    torch.manual_seed(4)
    layer = LoraLinear(torch.nn.Linear(8, 12, bias=False), r=4)
    with torch.no_grad():
        layer.lora_B.normal_(0, 0.1)
    x, res = torch.randn(3, 8), torch.randn(3, 12)
    full = layer(x)
    layer.disable_adapter()
    assert torch.allclose(layer(x, residual=res), layer.base_layer(x) + res)
    assert torch.allclose(layer(x, act="relu_sq"), torch.relu(layer.base_layer(x)) ** 2)
    layer.enable_adapter()
    layer.merge()
    assert torch.allclose(layer(x, residual=res), full + res, atol=1e-5)
    spec = layer.decode_spec()
    assert spec[1] is None and spec[0] is layer.base_layer.weight
    layer.unmerge()
    spec = layer.decode_spec()
    assert spec[1][0] is layer.lora_A and spec[1][2] == layer.scaling
