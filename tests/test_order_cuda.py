"""The eigenvalue-order kernel (column sums + stable descending argsort in one launch) against ``torch.argsort``."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("parts,n", [(1, 1), (1, 7), (2, 128), (1, 1000), (2, 8192), (4, 16384), (1, 20000)])
def test_order_matches_stable_descending_argsort(parts, n):
    from soap_tp_b200.engine import kernels as k

    g = torch.Generator().manual_seed(n)
    table = torch.randn(n, parts, generator=g).T.cuda()            # parts x n with unit stride along the parts
    if n > 16:
        table[:, 5] = table[:, 3]                                  # ties keep their index order
        table[:, n // 2] = table[:, 3]
    estimates = torch.zeros(n, device="cuda")
    for r in range(parts):                                         # the kernel adds the parts in index order
        estimates = estimates + table[r]
    expected = torch.argsort(estimates, descending=True, stable=True)
    order = k.order_by_estimate(table)
    assert order.dtype == torch.int64 and torch.equal(order, expected)


def test_order_puts_nan_estimates_last():
    from soap_tp_b200.engine import kernels as k

    values = torch.tensor([[1.0, float("nan"), 3.0, 2.0]], device="cuda")
    order = k.order_by_estimate(values)
    assert order.tolist()[:3] == [2, 3, 0] and order.tolist()[3] == 1
