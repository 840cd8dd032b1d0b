"""``adam_update`` against the closed form (cf. the reference's ``tests/unit/test_optimizer.py``)."""
import math

import pytest
import torch

from soap_tp_b200.ops import adam_update
from soap_tp_b200.utils.dense_soap import relative_l2

SHAPES = [(1, 1), (3, 5), (8, 8), (17, 9), (64, 33)]


def closed_form(g, m, v, step, b1, b2, eps):
    m2 = b1 * m + (1 - b1) * g
    v2 = b2 * v + (1 - b2) * g * g
    update = (m2 / (1 - b1**step)) / (v2.sqrt() / math.sqrt(1 - b2**step) + eps)
    return m2, v2, update


def check(device, shape, column_major, output_folder=None):
    torch.manual_seed(0)
    make = (lambda: torch.randn(shape[1], shape[0], dtype=torch.float64).T) if column_major else (
        lambda: torch.randn(shape, dtype=torch.float64))
    g, m, v = make(), make(), make().abs()
    em, ev, eu = closed_form(g, m, v, 3, 0.9, 0.99, 1e-6)
    g32, m32, v32 = (t.to(torch.float32).to(device) for t in (g, m, v))
    if column_major:
        g32, m32, v32 = (t.T.contiguous().T for t in (g32, m32, v32))
    out = adam_update(g32, m32, v32, 3, 0.9, 0.99, 1e-6)
    assert out.stride() == v32.stride()
    for got, want in ((m32, em), (v32, ev), (out, eu)):
        assert relative_l2(got, want) <= 1e-5
        torch.testing.assert_close(got.cpu().double(), want, rtol=1e-5, atol=1e-5)
    if output_folder is not None:
        with open(output_folder / "test_adam_l2.log", "a") as f:
            f.write(f"{shape[0]}x{shape[1]} {relative_l2(out, eu):.6e}\n")


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("column_major", [False, True])
def test_adam_cpu(shape, column_major, output_folder):
    check("cpu", shape, column_major, output_folder)


@pytest.mark.gpu
@pytest.mark.parametrize("shape", SHAPES + [(1000, 513)])
@pytest.mark.parametrize("column_major", [False, True])
def test_adam_cuda(shape, column_major):
    check("cuda", shape, column_major)


def test_adam_validation():
    t = torch.zeros(2, 2)
    with pytest.raises(ValueError):
        adam_update(t, t.clone(), t.clone(), 0)
    with pytest.raises(ValueError):
        adam_update(t, t.clone(), t.clone(), 1, beta1=1.0)
    with pytest.raises(ValueError):
        adam_update(t, t.clone(), t.clone(), 1, beta2=-0.1)
    with pytest.raises(ValueError):
        adam_update(t, t.clone(), t.clone(), 1, eps=0.0)
    with pytest.raises(ValueError):
        adam_update(t, torch.zeros(3, 2), t.clone(), 1)
