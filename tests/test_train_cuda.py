"""End-to-end training loop on the GPU: tensor-parallel Llama-shaped model + ``SoapTP`` on one device.

Exercises the optimizer's classification (SOAP for tagged 2-D weights, AdamW for the rest), the
device engine on many small parameters of different shapes in one step, refresh steps, and bf16
parameters with fp32 optimizer state.
"""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_tiny_llama_trains_with_soap_on_cuda():
    from soap_tp_b200 import train as train_module
    from soap_tp_b200.engine import kernels

    args = train_module.parse_args(["--preset", "tiny", "--steps", "8", "--precondition-frequency", "3",
                                    "--global-batch", "4", "--block-size", "16", "--lr", "1e-2"])
    summary = train_module.train(args)
    kernels.check_status()
    losses = summary["losses"]
    assert len(losses) == 8 and all(math.isfinite(v) for v in losses)
    # fresh random tokens every step: the loss cannot fall below log(vocabulary) = 4.16, and a working
    # optimizer keeps it from drifting upwards
    assert losses[-1] < losses[0] + 0.1 and abs(losses[0] - math.log(64)) < 0.5
