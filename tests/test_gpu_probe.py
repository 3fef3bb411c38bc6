"""The stand-alone hardware probes (csrc/rd_probe.cu) build and run: every probe ends with err 0."""

import subprocess

import pytest

from gpu_ragged_dot_b200 import probe


@pytest.mark.gpu
@pytest.mark.parametrize("which", ["sync", "pair", "mma"])
def test_probe_runs_clean(which):
    path = probe.build_probe()
    out = subprocess.run([path, which], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith(which)]
    assert lines, out.stdout
    assert all("err" not in ln or "err 0" in ln for ln in lines), out.stdout
    assert out.stdout.strip().splitlines()[-1] == "no error"
    if which == "mma":  # the tensor pipe's rate does not depend on the operand layout or the CTA group
        rates = [float(ln.split("complete ")[1].split(" clk")[0]) for ln in lines]
        assert max(rates) < 1.05 * min(rates), rates
