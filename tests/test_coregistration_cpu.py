"""This package next to the reference in one process (needs a checkout of the reference; skipped without).

The reference defines the ``uma_qmoe`` operators first; registering this package afterwards must keep the
reference's CPU correctness path and replace only the CUDA entries, and the reference's own pack reader must
register with this package's registry unchanged.  Runs in a child process because operator registrations
are global to the interpreter.
"""

import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def _reference_src() -> Path | None:
    for candidate in (os.environ.get("UMA_QMOE_REFERENCE"), str(ROOT.parent / "reference"), str(ROOT / "oracle" / "_ref")):
        if not candidate:
            continue
        for src in (Path(candidate) / "src", Path(candidate)):
            if (src / "uma_qmoe" / "custom_op.py").exists():
                return src
    return None


def test_registers_after_the_reference_and_takes_its_readers():
    src = _reference_src()
    if src is None:
        pytest.skip("no checkout of the reference")
    code = textwrap.dedent(f"""
        import sys
        sys.path.insert(0, {str(src)!r})
        sys.path.insert(0, {str(ROOT)!r})
        import numpy as np, torch
        from uma_qmoe import custom_op as ref_op
        from uma_qmoe.expert_pack import ExpertPackReader
        ref_op.register_moe_forward()                       # the reference defines the namespace ...
        from uma_qmoe_b200 import custom_op as op
        op.register_moe_forward()                           # ... this package adds its CUDA entries
        op.register_moe_forward()                           # idempotent
        reader = ExpertPackReader({str(ROOT / 'tests' / 'golden' / 'tiny.uqmoepk')!r})
        assert reader.mapping_count == 1
        mine = op.register_expert_pack(reader)              # the reference's reader, this package's registry
        with op.acquire_expert_pack(mine) as r:
            assert r is reader and op.expert_pack_for_handle(mine) is reader
        op.unregister_expert_pack(mine)
        # the reference's CPU correctness path still answers CPU calls
        theirs = ref_op.register_expert_pack(reader)
        x = torch.zeros(1, 2048, dtype=torch.bfloat16)
        idx = torch.zeros(1, 8, dtype=torch.int64)
        w = torch.zeros(1, 8)
        try:
            torch.ops.uma_qmoe.moe_forward(x, idx, w, 0, theirs, False)
            outcome = "ran"
        except Exception as exc:                            # the tiny pack has 4 x 256 tensors: a shape error from
            outcome = type(exc).__name__ + ": " + str(exc)  # the reference's own checks, not from this package
        assert "no cpu implementation is installed" not in outcome, outcome
        try:
            torch.ops.uma_qmoe.moe_forward(x, idx, w, 0, theirs, True)
            raise SystemExit("performance mode on CPU must fail closed")
        except RuntimeError as exc:
            assert "silent reference fallback is forbidden" in str(exc), exc
        ref_op.unregister_expert_pack(theirs)
        reader.close()
        print("coregistration ok:", outcome[:80])
    """)
    proc = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert "coregistration ok" in proc.stdout
