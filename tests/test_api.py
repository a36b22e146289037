"""Constructor contract of the four classes: same arguments, defaults, param-group keys and errors as
the reference (src/kaon/lion.py:152-208, src/kaon/adakaon.py:184-262, src/kaon/nekaon.py:100-182,
src/kaon/adamuon.py:196-262).  No GPU: nothing is stepped here."""
import pytest
import torch

import kaon_b200
from kaon_b200 import AdaMuon, Adakaon, Lion, Nekaon


def _params():
    g = torch.Generator().manual_seed(0)
    return [torch.nn.Parameter(torch.randn(4, 3, generator=g)), torch.nn.Parameter(torch.randn(5, generator=g))]


def test_exports():
    assert set(kaon_b200.__all__) >= {"Adakaon", "Nekaon", "Lion", "AdaMuon"}


@pytest.mark.parametrize("cls", [Lion, Adakaon, AdaMuon])
def test_invalid_args_rejected(cls):
    """reference tests/test_lion.py:307-318, tests/test_adamuon.py (test_invalid_args_rejected)"""
    for kw in (dict(momentum_dtype="2bit"), dict(betas=(1.0, 0.99)), dict(betas=(0.9, 1.0)), dict(lr=-1.0),
               dict(bf16_method="bogus")):
        with pytest.raises(ValueError):
            cls(_params(), **kw)


def test_lion_defaults_and_group_keys():
    opt = Lion(_params())
    g = opt.param_groups[0]
    assert g["lr"] == 1e-4 and g["betas"] == (0.9, 0.99) and g["weight_decay"] == 0.0
    assert g["momentum_dtype"] == "bfloat16" and g["momentum_4bit_block"] == 128
    assert g["cautious"] is True and g["gradient_centralization"] is True
    assert g["bf16_method"] == "stochastic_rounding"


def test_adakaon_defaults_and_group_keys():
    opt = Adakaon(_params())
    g = opt.param_groups[0]
    # exactly the reference's keys (src/kaon/adakaon.py:236-247)
    assert set(g) == {"params", "lr", "betas", "eps", "weight_decay", "clip_threshold", "momentum_dtype",
                      "momentum_4bit_block", "cautious", "gradient_centralization", "bf16_method"}
    assert g["clip_threshold"] == 1.0 and g["eps"] == (1e-30, 1e-3)


def test_per_group_overrides_are_kept():
    a, b = _params()
    opt = Adakaon([{"params": [a], "lr": 3e-4, "weight_decay": 0.2}, {"params": [b]}], lr=1e-4)
    assert opt.param_groups[0]["lr"] == 3e-4 and opt.param_groups[0]["weight_decay"] == 0.2
    assert opt.param_groups[1]["lr"] == 1e-4


def test_nekaon_preset_and_rejections():
    """reference tests/test_nekaon.py:55-66, 105-112"""
    opt = Nekaon(_params())
    assert opt.k == 1.5 and opt.rho == -1.5 and opt.norm == "none"
    g = opt.param_groups[0]
    assert g["weight_decay"] == 0.1 and g["betas"] == (0.5, 0.999) and g["momentum_dtype"] == "4bit"
    assert opt.base_optimizer is opt.inner and isinstance(opt.inner, Adakaon)
    with pytest.raises(ValueError):
        Nekaon(_params(), betas=(0.0, 0.999))
    with pytest.raises(ValueError):
        Nekaon(_params(), k=-1.0)
    with pytest.raises(TypeError):
        Nekaon([{"params": _params()}], low_vram_above=10)
    with pytest.raises(ValueError):
        Nekaon(_params(), low_vram_above=-1)


def test_nekaon_low_vram_above_builds_the_two_groups():
    """reference tests/test_nekaon.py:78-90: tensors above the threshold go to a momentum-free group at
    lr * low_vram_lr_ratio"""
    big, small = _params()
    opt = Nekaon([big, small], lr=1e-3, k=1.5, betas=(0.9, 0.999), momentum_dtype="float32", low_vram_above=10)
    assert len(opt.param_groups) == 2
    big_group = next(g for g in opt.param_groups if any(p is big for p in g["params"]))
    small_group = next(g for g in opt.param_groups if any(p is small for p in g["params"]))
    assert big_group["lr"] == 1e-3 * 0.5 and big_group["betas"] == (0.0, 0.999)
    assert small_group["lr"] == 1e-3 and small_group["betas"] == (0.9, 0.999)


def test_auto_lr_is_refused_loudly():
    with pytest.raises(NotImplementedError):
        Lion(_params(), auto_lr=True)


def test_step_without_gradients_is_a_no_op_even_on_cpu():
    opt = Lion(_params())
    opt.step()  # nothing has a gradient: no plan is built, no device is touched
    assert len(opt.state) == 0
