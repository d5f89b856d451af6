"""The twin-directory harness (csrc/zt_harness.cpp) against a directory written from the oracle in the
reference's wire format (src/cuda/attn_twin.zig:198-201,262-269; src/cuda/attn.cu:170-224)."""
import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HARNESS = os.path.join(ROOT, "z-transformer_b200", "zt_attn_harness")
sys.path.insert(0, os.path.join(ROOT, "oracle"))

SMALL = (("ctx256", 256, 4, 2, 32, 2000), ("odd-96-T40", 40, 8, 2, 96, 5))


def run(args, **env):
    e = dict(os.environ)
    e.update(env)
    return subprocess.run([HARNESS, *args], capture_output=True, text=True, env=e, timeout=600)


def test_list_reads_the_reference_wire_format(tmp_path):
    """No GPU: the manifest is parsed and every blob's size checked; a truncated blob and a missing manifest
    are refused the way attn.cu refuses them (attn.cu:170-224)."""
    import zt_twin
    assert os.path.exists(HARNESS), "build the library first (python -c 'import __graft_entry__ as g; g.build()')"
    d = str(tmp_path / "twin")
    zt_twin.write_twin_dir(d, SMALL, threads=2)
    r = run(["--list", d])
    assert r.returncode == 0, r.stderr
    lines = r.stdout.strip().splitlines()
    assert lines[0].startswith("ctx256 T=256 heads=4/2 head_dim=32 iters=2000")
    assert lines[1].startswith("odd-96-T40 T=40 heads=8/2 head_dim=96 iters=5")
    assert os.path.getsize(os.path.join(d, "ctx256.q.bin")) == 256 * 4 * 32 * 4
    assert os.path.getsize(os.path.join(d, "ctx256.dk.bin")) == 256 * 2 * 32 * 4
    with open(os.path.join(d, "ctx256.dv.bin"), "r+b") as f:
        f.truncate(100)
    r = run(["--list", d])
    assert r.returncode == 1 and "ctx256.dv.bin holds 100 bytes" in r.stderr
    r = run(["--list", str(tmp_path / "nothing")])
    assert r.returncode == 1 and "cannot open" in r.stderr
    assert run([]).returncode == 2


@pytest.fixture(scope="module")
def twin_dir(tmp_path_factory):
    import zt_twin
    d = str(tmp_path_factory.mktemp("twin"))
    zt_twin.write_twin_dir(d)  # the reference's eleven shapes
    return d


@pytest.mark.gpu
def test_harness_passes_the_reference_gates(twin_dir):
    """All eleven shapes of the reference's table through zt_attn_forward / zt_attn_backward: the forward
    within 1e-4, dq, dk, dv within 1e-5 (attn.cu:51,114), and the T = 8 launch of both entry points per shape."""
    r = run([twin_dir])
    sys.stdout.write(r.stdout)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "harness: PASS" in r.stdout
    assert r.stdout.count("forward 0  backward 0") == 11


@pytest.mark.gpu
def test_harness_negative_controls(twin_dir):
    """A gate that has never been seen to fail is not known to be a gate (run-attn.sh:126-177): each injected
    defect must fail the run, the four backward defects must leave four distinct signatures, and dropping
    the softmax Jacobian must leave dv exactly as the correct run reads it."""
    for variant in "1234":
        r = run([twin_dir], ZT_HARNESS_BROKEN=variant)
        assert r.returncode == 1, f"forward defect {variant} passed the gate\n{r.stdout}"
    good = run([twin_dir])
    assert good.returncode == 0

    def signature(out):
        m = re.search(r"max_abs_dq.*\n\s+ctx256\s+(\S+)\s+(\S+)\s+(\S+)", out)
        return m.groups()

    sigs = []
    for variant in "1234":
        r = run([twin_dir], ZT_HARNESS_BWD_BROKEN=variant)
        assert r.returncode == 1, f"backward defect {variant} passed the gate\n{r.stdout}"
        sigs.append(signature(r.stdout))
    assert len(set(sigs)) == 4, sigs
    assert sigs[2][2] == signature(good.stdout)[2], "dropping the Jacobian must not touch dv"
    assert run([twin_dir], ZT_HARNESS_BROKEN="7").returncode == 2


@pytest.mark.gpu
def test_harness_scale_relative_gate_at_training_scale(twin_dir):
    """dout five orders of magnitude smaller, as a training step supplies it (attn.cu:103-113): the backward is
    gated relative to max |ref| (attn_rel_tol, train.zig:706), and a defect is still caught at that scale."""
    r = run([twin_dir], ZT_HARNESS_DOUT_SCALE="1e-5")
    assert r.returncode == 0, r.stdout + r.stderr
    assert "of max |ref|" in r.stdout
    r = run([twin_dir], ZT_HARNESS_DOUT_SCALE="1e-5", ZT_HARNESS_BWD_BROKEN="3")
    assert r.returncode == 1


DEFECTS_HARNESS = os.path.join(ROOT, "z-transformer_b200", "zt_attn_harness_defects")


def run_defects(args, **env):
    e = dict(os.environ)
    e.update(env)
    return subprocess.run([DEFECTS_HARNESS, *args], capture_output=True, text=True, env=e, timeout=600)


@pytest.mark.gpu
def test_defects_compiled_into_the_kernels_are_caught(twin_dir):
    """The reference compiles defects into its kernels and requires its gates to fail on each of them
    (src/cuda/attn_kernels.cu:150-158,592-599,622-624; src/cuda/run-attn.sh:126-177).  The same here, for the
    defects that live inside a kernel and cannot be imitated through the ABI: a dropped causal mask and a skipped
    running-maximum correction in the forward (CUDA-core and tensor-core kernels alike), a dropped mask and a dropped
    softmax Jacobian in the backward.  The switches exist only in the library built with -DZT_DEFECTS, which only
    this harness binary links; with the switch at 0 that build passes every gate."""
    assert os.path.exists(DEFECTS_HARNESS), "build the library first"
    good = run_defects([twin_dir], ZT_HARNESS_KERNEL_DEFECT="0")
    assert good.returncode == 0, good.stdout + good.stderr

    def fwd_failures(out):
        table = out.split("backward against")[0]
        return len(re.findall(r"FAIL", table))

    def signature(out):
        m = re.search(r"max_abs_dq.*\n\s+ctx256\s+(\S+)\s+(\S+)\s+(\S+)", out)
        return m.groups()

    r = run_defects([twin_dir], ZT_HARNESS_KERNEL_DEFECT="1")
    assert r.returncode == 1, f"the dropped causal mask inside the kernels passed the gate\n{r.stdout}"
    assert "switched on" in r.stdout
    # The running maximum: these kernels move it lazily (only when it grows by more than 2^8), so on the reference's
    # fill, whose maximum settles in the first tile, there is no correction to skip.  A directory whose scores rise
    # with the key position makes every tile move it: correct kernel passes, the defect fails.
    import zt_twin
    rising = twin_dir + "-rising"
    zt_twin.write_twin_dir(rising, (("rise-32-T512", 512, 4, 2, 32, 5), ("rise-128-T256", 256, 8, 2, 128, 5),
                                    ("rise-256-T256", 256, 2, 1, 256, 5), ("rise-64-T100", 100, 4, 2, 64, 5)),
                           transform=zt_twin.rising_scores)
    # (gradients on this data are a few units, not the 0.03 the backward's absolute gate was calibrated on: the
    # backward is graded relative to max |ref| here, which ZT_HARNESS_DOUT_SCALE switches on)
    r = run_defects([rising], ZT_HARNESS_KERNEL_DEFECT="0", ZT_HARNESS_DOUT_SCALE="0.5")
    assert r.returncode == 0, r.stdout + r.stderr
    r = run_defects([rising], ZT_HARNESS_KERNEL_DEFECT="3", ZT_HARNESS_DOUT_SCALE="0.5")
    assert r.returncode == 1, f"the skipped running-maximum correction passed the gate\n{r.stdout}"
    assert fwd_failures(r.stdout) == 4, r.stdout  # tensor-core kernels (three widths) and the CUDA-core one
    sigs = {}
    for defect in ("11", "13"):
        r = run_defects([twin_dir], ZT_HARNESS_KERNEL_DEFECT=defect)
        assert r.returncode == 1, f"backward defect {defect} inside the kernels passed the gate\n{r.stdout}"
        sigs[defect] = signature(r.stdout)
    assert sigs["11"] != sigs["13"]
    assert sigs["13"][2] == signature(good.stdout)[2], "dropping the Jacobian must not touch dv"
    # the shipped library has no such switch: its harness refuses the request instead of pretending
    assert run([twin_dir], ZT_HARNESS_KERNEL_DEFECT="1").returncode == 2
    assert run_defects([twin_dir], ZT_HARNESS_KERNEL_DEFECT="5").returncode == 2
