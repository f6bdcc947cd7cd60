"""The drop-in on the reference's own caller: mako::gen::Session (the reference's src/gen/session.cpp, compiled
unmodified) runs its three decode loops over a stand-in engine twice — once linked with the reference's CPU sampler,
once with the header swap of oracle/dropin/shim and libmako_b200.so — and must generate the same tokens, make and
keep the same numbers of drafts, and reuse the same context on a second turn. The two programs are built where the
reference checkout is present (oracle/Makefile, target `dropin`) and travel as binaries; without them the test is
skipped."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_BIN = os.path.join(ROOT, "oracle", "_ref", "session_dropin_ref")
MAKO_BIN = os.path.join(ROOT, "oracle", "_ref", "session_dropin_mako")


def _env():
    """The CUDA runtime the library was linked against sits in the Python environment's package directories."""
    import torch
    dirs = [os.path.join(ROOT, "mako_b200"), os.path.join(os.path.dirname(torch.__file__), "lib")]
    try:
        import nvidia.cuda_runtime as rt
        dirs.append(os.path.join(list(rt.__path__)[0], "lib"))
    except Exception:
        pass
    env = dict(os.environ)
    env["LD_LIBRARY_PATH"] = ":".join(dirs + [env.get("LD_LIBRARY_PATH", "")])
    return env


def _have():
    return os.path.exists(REF_BIN) and os.path.exists(MAKO_BIN)


@pytest.mark.gpu
def test_reference_session_generates_the_same_tokens_on_the_gpu_sampler():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    if not _have():
        pytest.skip("the drop-in programs were not built (no reference checkout at build time)")
    want = subprocess.run([REF_BIN], capture_output=True, text=True, timeout=600)
    assert want.returncode == 0, want.stderr
    got = subprocess.run([MAKO_BIN], capture_output=True, text=True, timeout=600, env=_env())
    assert got.returncode == 0, got.stderr
    w, g = want.stdout.strip().splitlines(), got.stdout.strip().splitlines()
    assert len(w) == len(g) == 22
    for a, b in zip(w, g):
        assert a == b, f"\nreference: {a[:300]}\nmako_b200: {b[:300]}"
    # the scenarios did exercise the sampler: drafts were made, some kept and some rejected
    drafted = [line for line in w if " drafts=" in line and " drafts=0 " not in line]
    assert len(drafted) >= 6
    for line in drafted:
        f = dict(kv.split("=") for kv in line.split(" tokens=")[0].split()[1:])
        assert 0 < int(f["accepted"]) <= int(f["drafts"])


def test_dropin_program_has_no_cpu_path():
    """Without a GPU the program linked against libmako_b200.so fails with the library's message instead of
    sampling on the host; the reference build of the same driver runs."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    if not _have():
        pytest.skip("the drop-in programs were not built (no reference checkout at build time)")
    got = subprocess.run([MAKO_BIN], capture_output=True, text=True, timeout=600, env=_env())
    assert got.returncode != 0 and "no CUDA device" in got.stderr
    want = subprocess.run([REF_BIN], capture_output=True, text=True, timeout=600)
    assert want.returncode == 0 and len(want.stdout.strip().splitlines()) == 22
