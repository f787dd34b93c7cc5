"""Checks that need no GPU: the library loads and exports every symbol the
public headers declare, the C structs have the reference's layout, the host-only
parts of fg_sampler.h behave like the reference (golden vectors), and the
GPU-backed entry points fail loudly — not silently on a CPU path — when no CUDA
device is present."""
import ctypes
import json
import re
from ctypes import byref
from pathlib import Path

import numpy as np
import pytest
import torch

import flash_gordon_b200 as fg

ROOT = Path(__file__).resolve().parent.parent
GOLDEN = json.loads((Path(__file__).parent / "golden" / "sampler_golden.json").read_text())


def declared_functions() -> list[str]:
    names = []
    for header in sorted((ROOT / "include").glob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
        text = re.sub(r"^\s*#.*$", "", text, flags=re.M)
        for statement in text.split(";"):
            if "typedef" in statement or "{" in statement:
                continue
            found = re.search(r"\b(fg_[a-z0-9_]+)\s*\(", statement)
            if found:
                names.append(found.group(1))
    return sorted(set(names))


def test_every_declared_symbol_is_exported(library):
    names = declared_functions()
    assert len(names) >= 40, names
    missing = [name for name in names if not hasattr(library, name)]
    assert not missing, f"declared in include/ but not exported: {missing}"


def test_struct_layouts_match_the_reference_abi():
    assert ctypes.sizeof(fg.SamplerConfig) == 40          # include/fg_sampler.h:6-15 of the reference
    assert fg.SamplerConfig.seed.offset == 32
    assert ctypes.sizeof(fg.FgError) == 4 + 512           # include/fg.h:57-60 of the reference
    assert ctypes.sizeof(fg.SamplerState) == 8
    assert fg.SampleArgs.row_stride.offset == 24 and fg.SampleArgs.debug.offset == 96


def test_headers_compile_as_c17_and_agree_with_the_bindings(tmp_path):
    """A C17 translation unit that includes the public headers, built with the
    reference's warning flags, reports the struct layouts the ctypes mirror assumes."""
    import subprocess
    source = tmp_path / "probe.c"
    source.write_text("""
#include <stddef.h>
#include <stdio.h>
#include "fg_cuda_sampler.h"
int main(void) {
    printf("%zu %zu %zu %zu %zu %zu %zu\\n", sizeof(fg_sampler_config), offsetof(fg_sampler_config, seed),
           sizeof(fg_error), sizeof(fg_cuda_sample_args), offsetof(fg_cuda_sample_args, row_stride),
           offsetof(fg_cuda_sample_args, configs), offsetof(fg_cuda_sample_args, debug));
    return FG_ERR_INTERRUPTED == 9 && FG_ERR_ARGUMENT == 2 ? 0 : 1;
}
""")
    binary = tmp_path / "probe"
    subprocess.run(["gcc", "-std=c17", "-Wall", "-Wextra", "-Wpedantic", "-Werror", "-I", str(ROOT / "include"),
                    str(source), "-o", str(binary)], check=True)
    out = subprocess.run([str(binary)], check=True, capture_output=True, text=True).stdout.split()
    assert [int(x) for x in out] == [
        ctypes.sizeof(fg.SamplerConfig), fg.SamplerConfig.seed.offset, ctypes.sizeof(fg.FgError),
        ctypes.sizeof(fg.SampleArgs), fg.SampleArgs.row_stride.offset, fg.SampleArgs.configs.offset,
        fg.SampleArgs.debug.offset]


def test_presets_and_validation_table(library):
    cfg = fg.SamplerConfig()
    library.fg_sampler_config_defaults(byref(cfg))
    assert (cfg.temperature, cfg.top_k, cfg.repetition_penalty, cfg.seed) == (1.0, 20, 1.0, 0x9E3779B97F4A7C15)
    assert abs(cfg.top_p - 0.95) < 1e-7 and cfg.min_p == 0.0
    library.fg_sampler_config_greedy(byref(cfg))
    assert (cfg.temperature, cfg.top_p, cfg.top_k) == (0.0, 1.0, 1)
    library.fg_sampler_config_defaults(None)   # NULL is ignored, as in the reference
    for entry in GOLDEN["validate"]:
        v = entry["config"]
        cfg = fg.SamplerConfig(float(v[0]), float(v[1]), int(float(v[2])), float(v[3]), float(v[4]),
                               float(v[5]), float(v[6]), int(float(v[7])))
        err = fg.FgError()
        status = library.fg_sampler_config_validate(byref(cfg), byref(err))
        assert status == entry["status"], entry
        if status:
            assert err.code == fg.FG_ERR_ARGUMENT and err.text() == "invalid sampler controls"
    assert library.fg_sampler_config_validate(None, None) == fg.FG_ERR_ARGUMENT
    assert library.fg_sampler_penalties_active(None) is False
    assert library.fg_sampler_penalties_active(byref(fg.SamplerConfig.make(repetition=1.05)))
    assert not library.fg_sampler_penalties_active(byref(fg.SamplerConfig.make()))


def test_uniform_stream_matches_reference_bits(library):
    for entry in GOLDEN["uniform"]:
        got = np.array(fg.uniform_stream(entry["seed"], 16), dtype=np.float32).view(np.uint32)
        assert got.tolist() == entry["bits"]
    assert all(0.0 <= u < 1.0 for u in fg.uniform_stream(123, 1000))


def test_input_generator_draws_the_same_stream(library):
    """synth draws its uniforms without the native library; the bits must be the library's."""
    from flash_gordon_b200 import synth
    for seed in (0, 1, 123, 0x9E3779B97F4A7C15, 2**64 - 1):
        mine = np.array(synth.xorshift_uniforms(seed, 64), dtype=np.float32).view(np.uint32)
        theirs = np.array(fg.uniform_stream(seed, 64), dtype=np.float32).view(np.uint32)
        assert np.array_equal(mine, theirs), seed


def test_small_helpers(library):
    assert library.fg_align_up_u64(5, 4096) == 4096 and library.fg_align_up_u64(5, 0) == 5
    assert library.fg_is_aligned_u64(8192, 4096) and not library.fg_is_aligned_u64(1, 0)
    err = fg.FgError()
    library.fg_error_set.restype = None
    library.fg_error_set(byref(err), 4, b"token %u of %s", 7, b"row")
    assert err.code == 4 and err.text() == "token 7 of row"
    library.fg_error_set(None, 4, b"ignored")


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the behaviour without a GPU")
def test_no_silent_cpu_path_without_a_gpu(library):
    handle = ctypes.c_void_p()
    err = fg.FgError()
    assert library.fg_cuda_context_create(0, byref(handle), byref(err)) == fg.FG_ERR_UNAVAILABLE
    assert not handle.value and "CUDA" in err.text()
    from flash_gordon_b200.api import select
    status, _, _, _ = select(fg.SamplerConfig.make(), [1.0, 2.0], [1, 2], 0.5)
    assert status == fg.FG_ERR_UNAVAILABLE
    scores = (ctypes.c_float * 2)(1.0, 2.0)
    ids = (ctypes.c_uint32 * 2)(0, 1)
    counts = (ctypes.c_uint32 * 2)(1, 1)
    cfg = fg.SamplerConfig.make(presence=1.0)
    library.fg_sampler_apply_penalties(scores, ids, counts, 2, byref(cfg))
    assert list(scores) == [1.0, 2.0]                       # untouched: nothing ran on a CPU
    assert library.fg_sampler_last_status() == fg.FG_ERR_UNAVAILABLE
    with pytest.raises(fg.FgStatusError):
        fg.Context(0)


def test_missing_library_is_loud(monkeypatch, tmp_path):
    monkeypatch.setattr(fg, "_library", None)
    monkeypatch.setattr(fg, "LIBRARY_PATH", tmp_path / "libfgsampler.so")
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        fg.load_library()
