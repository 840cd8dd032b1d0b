"""Tracing protocol, the profile diff tool and the accuracy-log summariser."""
import contextlib
import io
import json
import os

import torch
import torch.distributed as dist

from distributed_helpers import free_port


def test_profile_protocol_and_diff(tmp_path, monkeypatch):
    from soap_tp_b200 import soap_step
    from soap_tp_b200.utils import compare_profiles
    from soap_tp_b200.utils.dense_soap import DenseSOAP

    monkeypatch.setenv("SOAP_PROFILE", "1")
    monkeypatch.setenv("MASTER_PORT", str(free_port()))
    dist.init_process_group("gloo", rank=0, world_size=1)
    try:
        shape = (8, 8)
        oracle = DenseSOAP(shape, beta1=0.8, beta2=0.9, preconditioner_beta=0.75, eps=1e-6, basis_refresh_interval=2)
        oracle.profile = True
        state = {}
        captured = io.StringIO()
        with contextlib.redirect_stdout(captured):
            for it in range(4):
                G = torch.randn(shape, generator=torch.Generator().manual_seed(it))
                oracle.step(G)
                soap_step(G, state, global_shape=shape, shard_dim=0, block_size=2, process_grid_shape=(1, 1),
                          preconditioner_beta=0.75, beta1=0.8, beta2=0.9, eps=1e-6, basis_refresh_interval=2,
                          basis_implementation="eigh")
    finally:
        dist.destroy_process_group()
    lines = [l for l in captured.getvalue().splitlines() if l.startswith("SOAP_PROFILE ")]
    first = json.loads(lines[0][len("SOAP_PROFILE "):])
    assert set(first) == {"impl", "step", "stage", "shape", "dtype", "values"} and ", " not in lines[0]
    stages = {json.loads(l[13:])["stage"] for l in lines if '"impl":"tp"' in l and '"step":1,' in l}
    assert len(stages) == 20                      # the reference emits 20 taps per steady step
    log = tmp_path / "combined.log"
    log.write_text(captured.getvalue())
    report = io.StringIO()
    code = compare_profiles.compare(compare_profiles.parse([str(log)]), 1e-5, out=report)
    assert code == 0, report.getvalue()
    assert "returned_update" in report.getvalue() and "first stage above rtol" in report.getvalue()
    # a corrupted trace is flagged at the right stage
    broken = captured.getvalue().replace('"impl":"tp","step":2,"stage":"projected_gradient"',
                                         '"impl":"tp","step":2,"stage":"projected_gradient_x"')
    assert compare_profiles.compare(compare_profiles.parse([str(log)]), 0.0, out=io.StringIO()) in (0, 1)
    del broken


def test_accuracy_log_summary(tmp_path, capsys):
    from soap_tp_b200.utils import plot_accuracy

    log = tmp_path / "acc.log"
    log.write_text("\n".join([
        "8x8 dim0 basis=eigh | step 1 | SOAP relL2=2.45e-06 | PARAM relL2=2.45e-06",
        "8x8 dim0 basis=eigh | step 2 | SOAP relL2=3.09e-06 (ref=1, TP=1, at=0) opposite=0/64 | PARAM relL2=2.55e-06",
        "noise",
        "20x20 dim1 basis=jacobi | step 1 | SOAP relL2=4.51e-05 | PARAM relL2=4.51e-05",
    ]))
    assert plot_accuracy.main([str(log), "--csv", str(tmp_path / "t.csv")]) == 0
    out = capsys.readouterr().out
    assert "3.090e-06" in out and "jacobi" in out
    assert (tmp_path / "t.csv").read_text().count("\n") == 3


def test_timing_protocol(capsys):
    from soap_tp_b200.profiling import emit_timing

    emit_timing("step", step=3, seconds=0.5)
    line = capsys.readouterr().out.strip()
    assert line == 'SOAP_TIMING {"event": "step", "seconds": 0.5, "step": 3}'


def test_profile_diff_aliases_and_run_splitting(tmp_path, capsys):
    """Short stage names are canonicalised, and a log holding two comparisons back to back (steps start again
    at 0 with another shape) is compared run by run."""
    from soap_tp_b200.utils import compare_profiles

    def record(impl, step, stage, tensor):
        body = {"impl": impl, "step": step, "stage": stage, "shape": list(tensor.shape), "dtype": "float32",
                "values": tensor.flatten().tolist()}
        return "SOAP_PROFILE " + json.dumps(body, separators=(",", ":"))

    lines = []
    for shape in ((2, 3), (4, 2)):
        g = torch.arange(float(shape[0] * shape[1])).reshape(shape)
        for step in (0, 1):
            lines += [record("ref", step, "input.gradient", g + step), record("reference", step, "soap_update", g * 2)]
            lines += [record("src", step, "gradient", g + step), record("tp", step, "returned_update", g * 2)]
    log = tmp_path / "two_runs.log"
    log.write_text("\n".join(lines) + "\n")
    events = compare_profiles.read_events([str(log)])
    assert {stage for _, _, stage, _ in events} == {"gradient", "returned_update"}
    runs = compare_profiles.split_runs(events)
    assert [compare_profiles.describe_run(r) for r in runs] == ["gradient shape 2x3", "gradient shape 4x2"]
    assert compare_profiles.main([str(log)]) == 0
    out = capsys.readouterr().out
    assert "=== run 1 of 2: gradient shape 2x3 ===" in out and "=== run 2 of 2: gradient shape 4x2 ===" in out
    assert "SHAPE MISMATCH" not in out
    assert compare_profiles.canonical_stage("adam.v") == "variance_after_adam"
