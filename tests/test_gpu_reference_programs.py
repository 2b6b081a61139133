"""C-ML's own test programs for the path (tests/test_gguf_quant.c, test_qlora.c, test_lora.c,
test_tensor_parallel.c, test_paged_attention.c of its tree), compiled unchanged against this
repo's include/ and linked to libcml_b200.so by `make -C oracle reftests` where the C-ML tree is
present. The binaries travel with the build; here they run on the GPU and every case in them must
pass. (test_speculative.c and test_serving.c need no device and run in the CPU suite.)"""
import re
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
BIN = ROOT / "oracle" / "_ref" / "tests"
pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["test_gguf_quant", "test_qlora", "test_lora", "test_tensor_parallel", "test_paged_attention"])
def test_reference_program_passes_against_this_library(name, torch_dev):
    exe = BIN / name
    if not exe.exists():
        pytest.skip("reference test programs were not built (no C-ML tree at build time)")
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300, cwd=str(ROOT))
    out = r.stdout + r.stderr
    assert r.returncode == 0, out[-3000:]
    m = re.search(r"(\d+)/(\d+) (?:tests )?passed", out)
    if m:
        assert m.group(1) == m.group(2) and int(m.group(2)) > 0, out[-3000:]
    else:
        assert "passed" in out and "FAIL" not in out, out[-3000:]
