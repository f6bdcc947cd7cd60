"""CPU tests of the boundary: the C-ABI library loads, exports every symbol the public header declares, validates
arguments like the reference does, and refuses to run without a GPU instead of computing anything on the host."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "mako_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mk_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from mako_b200 import lib
    names = declared_functions()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/mako_b200.h but not exported"


def test_version_string_names_the_architecture():
    import mako_b200
    assert "sm_100a" in mako_b200.version()


def test_check_sampling_ranges():
    """The reference's upstream checks (src/server/openai.cpp:316-328; pinned by tests/server_test.cpp:312-317)."""
    from mako_b200 import SamplingParams, check_sampling
    check_sampling(SamplingParams())
    check_sampling(SamplingParams(temperature=0.0))
    check_sampling(SamplingParams(temperature=1e-3, repetition_penalty=100.0, presence_penalty=-100.0))
    for bad in [SamplingParams(temperature=5e-4), SamplingParams(repetition_penalty=0.0),
                SamplingParams(repetition_penalty=100.5), SamplingParams(presence_penalty=101.0),
                SamplingParams(frequency_penalty=-100.5), SamplingParams(top_p=float("nan")),
                SamplingParams(min_p=float("inf"))]:
        with pytest.raises(ValueError):
            check_sampling(bad)


def test_empty_vocabulary_is_invalid_argument():
    """Sampler::Sampler throws std::invalid_argument for n_vocab == 0 (src/gen/sampler.cpp:11-12)."""
    from mako_b200 import lib
    h = C.c_void_p()
    assert lib.mk_sampler_create(C.byref(h), 0, 0, 1) == 1
    assert b"empty vocabulary" in lib.mk_last_error()
    from mako_b200 import BatchSampler, Sampler, SamplingParams
    with pytest.raises(ValueError):
        BatchSampler(0, 1)
    with pytest.raises(ValueError):
        Sampler(SamplingParams(), 0, 1)


def test_no_cpu_fallback():
    """Without a CUDA device the library reports MK_ERR_NO_DEVICE; it never computes on the host."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from mako_b200 import BatchSampler, MakoError
    with pytest.raises(MakoError) as e:
        BatchSampler(1000, 4)
    assert e.value.code == 4


def test_row_bytes_formula():
    """4V + 4H + 4*ceil(V/32) [mask] + 8*n_bias + 4*n_uniforms + 8 (token + probability out)."""
    from mako_b200 import lib
    assert lib.mk_row_bytes(151552, 0, 0, 0, 1) == 606220
    assert lib.mk_row_bytes(129280, 4096, 0, 0, 1) == 533516
    assert lib.mk_row_bytes(151552, 0, 1, 64, 1) == 625676


def test_product_does_not_import_the_oracle():
    """Nothing under mako_b200/ may import, load or execute the CPU checkers."""
    pkg = os.path.join(ROOT, "mako_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in src.lower(), f"{f} mentions the oracle"


def test_cpp_header_compiles_and_mirrors_the_reference_errors(tmp_path):
    """include/mako_b200/sampler.hpp: same constructor signature as the reference class; an empty vocabulary throws
    std::invalid_argument (src/gen/sampler.cpp:11-12) before any device is touched."""
    import subprocess
    src = tmp_path / "t.cpp"
    src.write_text(
        '#include <mako_b200/sampler.hpp>\n#include <cstdio>\n'
        'int main() { using namespace mako_b200::gen; SamplingParams p; p.temperature = 0.7f; p.top_k = 40;\n'
        '  try { Sampler s(p, 0, 1); } catch (const std::invalid_argument& e) { std::puts(e.what()); return 0; }\n'
        '  return 1; }\n')
    exe = tmp_path / "t"
    lib_dir = os.path.join(ROOT, "mako_b200")
    subprocess.check_call(["g++", "-std=c++20", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe),
                           "-L", lib_dir, "-lmako_b200", f"-Wl,-rpath,{lib_dir}", "-Wl,--allow-shlib-undefined"])
    import torch  # its CUDA wheels carry libcudart; expose it to the child
    cudart = [os.path.join(os.path.dirname(torch.__file__), "..", "nvidia", "cuda_runtime", "lib")]
    env = dict(os.environ, LD_LIBRARY_PATH=":".join(cudart + [os.environ.get("LD_LIBRARY_PATH", "")]))
    out = subprocess.run([str(exe)], env=env, capture_output=True, text=True)
    assert out.returncode == 0 and "empty vocabulary" in out.stdout
