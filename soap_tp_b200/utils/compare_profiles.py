#!/usr/bin/env python3
"""Diff ``SOAP_PROFILE`` value traces of two SOAP implementations stage by stage.

    python -m soap_tp_b200.utils.compare_profiles oracle.log tp.log [--rtol 1e-5]
    python -m soap_tp_b200.utils.compare_profiles combined.log

Input lines look like ``SOAP_PROFILE {"impl": "reference"|"tp", "step": k, "stage": ..., "shape":
[...], "values": [...]}``; anything else in a log is skipped.  Traces come from
``SOAP_PROFILE=1`` runs of :func:`soap_tp_b200.soap_step` (``impl: "tp"``) and of
:class:`soap_tp_b200.utils.dense_soap.DenseSOAP` (``impl: "reference"``); logs written by the
reference project use the same protocol (``src/soap_tp/soap.py:39-57``,
``tests/reference/soap.py:14-45``) and can be mixed in.

Stage names are canonicalised first: the short names used by earlier instrumentation of the reference
(``input.gradient``, ``adam.m``, ``soap_update``, ``left_basis_next`` ...; the reference's table is
``scripts/compare_soap_profiles.py:35-79``) map onto the names this package writes.  A log that holds several
comparisons one after the other (a parametrised test run: every shape writes its own trace with steps
starting again at 0) is split into runs, each compared by itself (``scripts/compare_soap_profiles.py:227-253``):
a new run starts at a ``gradient`` record whose (implementation, step) was already seen once both
implementations have written something.

Eigenvectors are defined up to sign.  For every step the tool derives one sign per basis column
from the two ``left_basis`` / ``right_basis`` tensors and applies it to every tensor that lives in
rotated coordinates (projected gradient, momentum, coordinate update) before comparing, as the
reference's ``scripts/compare_soap_profiles.py:298-411`` does; the variance is sign-free and
parameter-space tensors are compared as they are.  Reported per stage: relative L2 error, number of
entries with strictly opposite sign, and the first stage that is not bit-identical / exceeds
``--rtol``.
"""
from __future__ import annotations

import argparse
import json
import sys
from collections import OrderedDict, defaultdict
from typing import Dict, Iterable, List, Optional, Tuple

import torch

PREFIX = "SOAP_PROFILE "
IMPLEMENTATION_NAMES = {"reference": "reference", "ref": "reference", "tp": "tp", "src": "tp", "source": "tp",
                        "soap-tp": "tp", "soap_tp": "tp"}
STAGES = [
    "gradient", "left_preconditioner", "right_preconditioner", "left_basis", "right_basis",
    "momentum_before_adam", "variance_before_adam", "gradient_2d", "projected_gradient",
    "momentum_after_adam", "variance_after_adam", "coordinate_update", "backrotated_update", "returned_update",
    "left_preconditioner_after_step", "right_preconditioner_after_step", "left_basis_after_step",
    "right_basis_after_step", "momentum_after_step", "variance_after_step", "parameter_after_step",
]
# other spellings of the same taps -> the names above
STAGE_ALIASES = {
    "input.gradient": "gradient", "grad": "gradient",
    "preconditioner.ema.0": "left_preconditioner", "preconditioner.ema.1": "right_preconditioner",
    "basis.initial.output.0": "left_basis", "basis.initial.output.1": "right_basis",
    "adam.m": "momentum_after_adam", "momentum": "momentum_after_adam",
    "adam.v": "variance_after_adam", "variance": "variance_after_adam",
    "projected_update": "coordinate_update", "soap_update": "returned_update", "update": "returned_update",
    "left_preconditioner_next": "left_preconditioner_after_step",
    "right_preconditioner_next": "right_preconditioner_after_step",
    "left_basis_next": "left_basis_after_step", "right_basis_next": "right_basis_after_step",
    "momentum_next": "momentum_after_step", "variance_next": "variance_after_step",
    "parameter.after": "parameter_after_step",
}


def canonical_stage(name: str) -> str:
    return STAGE_ALIASES.get(name, name)


# stage -> which basis pair its coordinates refer to ("now": bases used by the step, "next": refreshed bases)
ROTATED = {"projected_gradient": "now", "momentum_before_adam": "now", "momentum_after_adam": "now",
           "coordinate_update": "now", "momentum_after_step": "next"}
BASES = {"left_basis": ("now", 0), "right_basis": ("now", 1), "left_basis_after_step": ("next", 0),
         "right_basis_after_step": ("next", 1)}


def read_events(paths: Iterable[str]) -> List[Tuple[str, int, str, torch.Tensor]]:
    """Every ``SOAP_PROFILE`` record of the logs, in file order: ``(implementation, step, stage, tensor)``."""
    events: List[Tuple[str, int, str, torch.Tensor]] = []
    for path in paths:
        stream = sys.stdin if path == "-" else open(path)
        with stream:
            for line in stream:
                position = line.find(PREFIX)
                if position < 0:
                    continue
                try:
                    record = json.loads(line[position + len(PREFIX):])
                except json.JSONDecodeError:
                    continue
                impl = IMPLEMENTATION_NAMES.get(str(record.get("impl", "")).lower())
                if impl is None:
                    continue
                payload = record.get("tensor", record)
                tensor = torch.tensor(payload["values"], dtype=torch.float64).reshape(payload["shape"])
                events.append((impl, int(record["step"]), canonical_stage(str(record["stage"])), tensor))
    return events


def split_runs(events) -> List[list]:
    """Cut a log that holds several comparisons back to back into one event list per comparison."""
    runs: List[list] = []
    current: list = []
    seen, writers = set(), set()
    for event in events:
        impl, step, stage, _ = event
        if stage == "gradient" and (impl, step, stage) in seen and writers == {"reference", "tp"}:
            runs.append(current)
            current, seen, writers = [], set(), set()
        current.append(event)
        seen.add((impl, step, stage))
        writers.add(impl)
    if current:
        runs.append(current)
    return runs


def traces_of(events) -> Dict[str, Dict[int, "OrderedDict[str, torch.Tensor]"]]:
    traces: Dict[str, Dict[int, OrderedDict]] = {"reference": defaultdict(OrderedDict), "tp": defaultdict(OrderedDict)}
    for impl, step, stage, tensor in events:
        traces[impl][step][stage] = tensor
    return traces


def parse(paths: Iterable[str]) -> Dict[str, Dict[int, "OrderedDict[str, torch.Tensor]"]]:
    """All records of the logs as one comparison (logs with a single run)."""
    return traces_of(read_events(paths))


def describe_run(events) -> str:
    for impl, step, stage, tensor in events:
        if stage == "gradient":
            return "gradient shape " + "x".join(str(d) for d in tensor.shape)
    return f"{len(events)} records"


def column_signs(candidate: torch.Tensor, target: torch.Tensor) -> Tuple[torch.Tensor, float]:
    dots = (candidate * target).sum(dim=0)
    signs = torch.where(dots < 0, -torch.ones_like(dots), torch.ones_like(dots))
    return signs, float(dots.abs().min()) if dots.numel() else 1.0


def compare(traces, rtol: float, out=sys.stdout) -> int:
    reference, tp = traces["reference"], traces["tp"]
    steps = sorted(set(reference) & set(tp))
    if not steps:
        print("no common steps between the two traces", file=out)
        return 2
    failures = 0
    for step in steps:
        signs: Dict[Tuple[str, int], torch.Tensor] = {}
        for stage, (when, axis) in BASES.items():
            if stage in reference[step] and stage in tp[step]:
                signs[(when, axis)], weakest = column_signs(tp[step][stage], reference[step][stage])
                flipped = int((signs[(when, axis)] < 0).sum())
                print(f"step {step:3d} {stage:32s} aligned {flipped} flipped columns, weakest |dot| {weakest:.3e}", file=out)
        first_inexact: Optional[str] = None
        first_failing: Optional[str] = None
        names = [s for s in STAGES if s in reference[step] and s in tp[step]]
        names += sorted((set(reference[step]) & set(tp[step])) - set(STAGES))
        for stage in names:
            expected, actual = reference[step][stage], tp[step][stage]
            if expected.shape != actual.shape:
                print(f"step {step:3d} {stage:32s} SHAPE MISMATCH {tuple(expected.shape)} vs {tuple(actual.shape)}", file=out)
                failures += 1
                continue
            if stage in BASES:
                actual = actual * signs[BASES[stage]]
            elif stage in ROTATED:
                when = ROTATED[stage]
                if (when, 0) in signs:
                    actual = actual * signs[(when, 0)][:, None]
                if (when, 1) in signs:
                    actual = actual * signs[(when, 1)][None, :]
            norm = float(expected.norm())
            error = float((actual - expected).norm()) / norm if norm > 0 else float(actual.norm())
            opposite = int(((actual * expected) < 0).sum())
            exact = bool(torch.equal(actual, expected))
            verdict = "ok" if error <= rtol else "FAIL"
            if not exact and first_inexact is None:
                first_inexact = stage
            if error > rtol and first_failing is None:
                first_failing = stage
                failures += 1
            print(f"step {step:3d} {stage:32s} relL2={error:.3e} opposite={opposite}/{expected.numel()} "
                  f"{'bit-identical' if exact else verdict}", file=out)
        print(f"step {step:3d} first non-bit-identical stage: {first_inexact}; first stage above rtol {rtol:g}: {first_failing}",
              file=out)
    return 1 if failures else 0


def main(argv: Optional[List[str]] = None) -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("logs", nargs="+", help="one or two log files ('-' for stdin)")
    parser.add_argument("--rtol", type=float, default=1e-5)
    args = parser.parse_args(argv)
    runs = split_runs(read_events(args.logs))
    if len(runs) <= 1:
        return compare(traces_of(runs[0] if runs else []), args.rtol)
    worst = 0
    for index, events in enumerate(runs):
        print(f"=== run {index + 1} of {len(runs)}: {describe_run(events)} ===")
        worst = max(worst, compare(traces_of(events), args.rtol))
    return worst


if __name__ == "__main__":
    raise SystemExit(main())
