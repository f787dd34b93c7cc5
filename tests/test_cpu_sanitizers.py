"""The host-only C of the library -- wire codecs, logit dump, request parser -- compiled with
AddressSanitizer and UndefinedBehaviorSanitizer and driven with random and damaged inputs
(tests/sanitize/fuzz_host.c).  The GPU pool offers no compute-sanitizer, so the host parts get
the sanitizers, and the device parts get exhaustive small cases against the oracle instead.
fg_sampler_config_validate / _defaults and fg_error_set come from the oracle's port here: the
library's own live beside code that talks to the GPU."""
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HOST = ROOT / "flash_gordon_b200" / "csrc" / "host"


def test_host_codecs_and_parser_under_asan_and_ubsan(tmp_path):
    if shutil.which("gcc") is None:
        pytest.skip("no C compiler")
    binary = tmp_path / "fuzz_host"
    build = subprocess.run(
        ["gcc", "-std=c17", "-D_GNU_SOURCE", "-O1", "-g", "-fsanitize=address,undefined",
         "-fno-sanitize-recover=all", "-fno-omit-frame-pointer", "-Wall", "-Wextra", "-Werror",
         "-I", str(ROOT / "include"), "-I", str(HOST),
         str(ROOT / "tests" / "sanitize" / "fuzz_host.c"), str(HOST / "fg_output_wire.c"), str(HOST / "fg_request.c"),
         str(ROOT / "oracle" / "fg_sampler_port.c"), "-lm", "-o", str(binary)],
        capture_output=True, text=True)
    if build.returncode != 0 and "sanitize" in build.stderr and "cannot find" in build.stderr:
        pytest.skip("the sanitizer runtimes are not installed")
    assert build.returncode == 0, build.stderr
    run = subprocess.run([str(binary)], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, run.stdout + run.stderr
    assert "accepted" in run.stdout
