"""CPU-side checks of the drop-in boundary: the C-ABI library loads, exports every symbol the
public headers declare, rejects bad arguments without touching a GPU, and the host repack is
a byte-exact bijection."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]


def _declared_functions():
    names = []
    for h in sorted((ROOT / "include").glob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", h.read_text(), flags=re.S)
        text = re.sub(r"//[^\n]*", "", text)
        for m in re.finditer(r"\b([A-Za-z_][A-Za-z0-9_]*)\s*\([^;{}()]*(?:\([^()]*\)[^;{}()]*)*\)\s*;", text):
            name = m.group(1)
            if name not in ("defined", "sizeof", "__attribute__"):
                names.append(name)
    return sorted(set(names))


def test_library_exports_every_declared_symbol(pkg):
    names = _declared_functions()
    assert len(names) >= 25
    missing = [n for n in names if not hasattr(pkg.lib, n)]
    assert not missing, f"declared in include/*.h but not exported: {missing}"


@pytest.mark.parametrize("qtype,bb", [(7, 34), (2, 18)])
def test_repack_is_a_bijection(pkg, synth, qtype, bb):
    rng = np.random.default_rng(5)
    rows, cols = 37, 96                       # ragged row count, three blocks per row
    blocks = (synth.q8_0_blocks if qtype == 7 else synth.q4_0_blocks)(rng, rows, cols)
    qs, sc = pkg.repack_gguf(qtype, blocks, rows, cols)
    assert qs.size == rows * cols * (1 if qtype == 7 else 0.5) and sc.size == rows * (cols // 32) * 2
    back = np.zeros_like(blocks)
    pkg.check(pkg.lib.cmlb200_unrepack_gguf(qtype, pkg.np_ptr(qs), pkg.np_ptr(sc), rows, cols, pkg.np_ptr(back)))
    assert np.array_equal(back, blocks)
    b2 = blocks.reshape(-1, bb)
    assert np.array_equal(sc.reshape(-1, 2), b2[:, :2]) and np.array_equal(qs.reshape(-1, bb - 2), b2[:, 2:])


def test_repack_rejects_bad_arguments(pkg):
    buf = np.zeros(1024, np.uint8)
    p = pkg.np_ptr(buf)
    assert pkg.lib.cmlb200_repack_gguf(7, None, 1, 32, p, p) == -1
    assert pkg.lib.cmlb200_repack_gguf(7, p, 1, 33, p, p) == -1          # cols % 32
    assert pkg.lib.cmlb200_repack_gguf(100, p, 1, 32, p, p) == -1        # NF4 is not a GGUF block type
    assert b"cols" in pkg.last_error() or b"type" in pkg.last_error()
    assert pkg.lib.cmlb200_qs_bytes(2, 4, 64, 32) == 128 and pkg.lib.cmlb200_scale_bytes(2, 4, 64, 32) == 16
    assert pkg.lib.cmlb200_qs_bytes(100, 4, 64, 64) == 128 and pkg.lib.cmlb200_scale_bytes(100, 4, 64, 64) == 16
    assert pkg.lib.cmlb200_qs_bytes(55, 4, 64, 32) == 0


def test_compute_entry_points_validate_before_launching(pkg):
    """Argument checks mirror C-ML's (-1 / NULL on NULL pointers, numel == 0, unknown type,
    numel % block != 0) and run before any CUDA call, so they hold without a GPU."""
    lib = pkg.lib
    fake = 0x1000
    assert lib.cmlb200_gguf_dequantize(7, None, fake, 32, None) == -1
    assert lib.cmlb200_gguf_dequantize(7, fake, fake, 0, None) == -1
    assert lib.cmlb200_gguf_dequantize(12, fake, fake, 128, None) == -1          # Q4_K blocks hold 256 elements
    assert lib.cmlb200_gguf_dequantize(6, fake, fake, 256, None) == -1           # not a type C-ML reads
    assert lib.cmlb200_gguf_dequantize(2, fake, fake, 48, None) == -1
    assert lib.cmlb200_dequantize_nf4(fake, fake, 0, 64, 64, fake, None) == -1
    W = pkg.QMat(pkg.Q4_0, 8, 48, 32, fake, fake)            # cols not a multiple of 32
    assert lib.cmlb200_gemv(W, fake, fake, 1, None) == -1
    W = pkg.QMat(pkg.Q4_0, 8, 64, 32, fake, fake)
    assert lib.cmlb200_gemv(W, fake, fake, 33, None) == -1     # outside the decode range
    assert lib.cmlb200_gemv(W, None, fake, 1, None) == -1
    W = pkg.QMat(pkg.NF4, 8, 64, 48, fake, fake)             # NF4 block must divide cols
    assert lib.cmlb200_gemv(W, fake, fake, 1, None) == -1
    W = pkg.QMat(pkg.Q4_0, 8, 80, 32, fake, fake)            # cols must be a multiple of 32
    assert lib.cmlb200_gemm_bf16(W, fake, fake, 64, None) == -1
    assert lib.cmlb200_gemm_bf16(pkg.QMat(pkg.Q4_0, 8, 128, 32, fake, fake), fake, fake, 0, None) == -1


@pytest.mark.parametrize("qtype", [7, 2])
def test_tile_major_repack_is_a_bijection(pkg, synth, qtype):
    rng = np.random.default_rng(6)
    rows, cols = 200, 256                     # two row tiles, the second partial
    blocks = (synth.q8_0_blocks if qtype == 7 else synth.q4_0_blocks)(rng, rows, cols)
    tiles = pkg.repack_tiles(qtype, blocks, rows, cols)
    unit = 4352 if qtype == 7 else 2304
    assert tiles.size == unit * 2 * (cols // 32)
    back = np.zeros_like(blocks)
    pkg.check(pkg.lib.cmlb200_unrepack_tiles(qtype, pkg.np_ptr(tiles), rows, cols, pkg.np_ptr(back)))
    assert np.array_equal(back, blocks)
    assert pkg.lib.cmlb200_repack_tiles(qtype, pkg.np_ptr(blocks), rows, 48, pkg.np_ptr(tiles)) == -1
    assert pkg.lib.cmlb200_tiles_bytes(100, rows, cols) == 0


def test_library_exports_nothing_but_the_declared_symbols(pkg):
    """The shared library is linked with a version script made from include/*.h: internal helpers
    (NCCL shim, GGUF internals, kernel launchers) are not part of the ABI."""
    import subprocess
    out = subprocess.run(["nm", "-D", "--defined-only", str(ROOT / "c-ml_b200" / "lib" / "libcml_b200.so")], capture_output=True, text=True, check=True).stdout
    exported = {line.split()[-1] for line in out.splitlines() if line.strip()}
    declared = set(_declared_functions()) | {"g_log_level", "CML_NF4_TABLE"}
    assert exported <= declared, sorted(exported - declared)


def test_init_cleanup_and_seed_are_reference_counted_no_ops(pkg):
    """cml_init / cml_cleanup (C-ML src/cml.c:376-440) and tensor_manual_seed
    (include/tensor/tensor.h:143), which examples/llama_inference.c:79-83 calls before anything else."""
    import ctypes as C
    lib = pkg.lib
    lib.tensor_manual_seed.argtypes = [C.c_uint64]
    lib.tensor_get_seed.restype = C.c_uint64
    assert lib.cml_cleanup() == 0                      # without a matching init: nothing happens
    assert lib.cml_init() == 0 and lib.cml_init() == 0
    lib.tensor_manual_seed(1234567890123)
    assert lib.tensor_get_seed() == 1234567890123
    assert lib.cml_cleanup() == 0 and lib.cml_cleanup() == 0


def test_sampling_branch_matches_the_compiled_reference(pkg, ob, ref, golden):
    """cml_llama_sample_token (src/nn/llama.c:627-737): temperature, descending sort, top-k softmax,
    top-p cut, renormalisation and one rand() draw. Host code, so it runs without a GPU; the C
    library generator is seeded exactly as the reference wrapper seeded it."""
    import ctypes as C
    libc = C.CDLL(None)
    logits = np.ascontiguousarray(golden["sample_logits"])
    t = pkg.numpy_to_tensor(logits)
    try:
        for (temp, top_p, top_k, do_sample, seed), want in zip(golden["sample_cases"], golden["sample_ids"]):
            cfg = pkg.GenerationConfig(float(temp), float(top_p), int(top_k), 16, 2, bool(do_sample))
            libc.srand(int(seed))
            got = pkg.lib.cml_llama_sample_token(t, C.byref(cfg))
            assert got == int(want), (temp, top_p, top_k, do_sample, seed, got, int(want))
            if ref is not None:
                assert ref.ref_sample_token(ob.p(logits), 2, logits.shape[1], float(temp), float(top_p), int(top_k), int(do_sample), int(seed)) == got
        greedy = pkg.GenerationConfig(0.8, 0.9, 40, 16, 2, False)
        assert pkg.lib.cml_llama_sample_token(t, C.byref(greedy)) == 17          # first of two equal maxima
        assert pkg.lib.cml_llama_sample_token(None, C.byref(greedy)) == -1
    finally:
        pkg.lib.tensor_free(t)


def test_generate_needs_loaded_weights_and_a_tokenizer(pkg):
    import ctypes as C
    cfg = pkg.LlamaConfig(64, 64, 128, 1, 2, 2, 16, 10000.0, 1e-5, 0, 0)
    m = pkg.lib.cml_llama_create(C.byref(cfg))
    assert m
    pkg.lib.cml_set_log_level(4)
    gen = pkg.lib.cml_generation_default_config()
    assert not pkg.lib.cml_llama_generate(m, b"hello", C.byref(gen))            # weights not loaded
    assert not pkg.lib.cml_llama_generate(None, b"hello", C.byref(gen))
    pkg.lib.cml_set_log_level(3)
    pkg.lib.cml_llama_free(m)


def test_reference_example_program_links_against_the_library(pkg, ob, tmp_path):
    """examples/llama_inference.c of the C-ML tree, unmodified, compiles against include/ (through the
    forwarding cml.h and nn/llama.h) and links against libcml_b200.so alone."""
    import subprocess
    root = ob.reference_root()
    if root is None:
        pytest.skip("the C-ML source tree is not on this machine")
    exe = tmp_path / "llama_inference"
    libdir = ROOT / "c-ml_b200" / "lib"
    cmd = ["gcc", "-std=c11", "-D_POSIX_C_SOURCE=200809L", f"-I{ROOT / 'include'}", str(Path(root) / "examples" / "llama_inference.c"),
           "-o", str(exe), f"-L{libdir}", "-lcml_b200", f"-Wl,-rpath,{libdir}", "-lm"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([str(exe), "-h"], capture_output=True, text=True)
    assert r.returncode == 0 and "LLaMA inference" in r.stdout
    r = subprocess.run([str(exe), str(tmp_path / "missing.gguf"), "--greedy"], capture_output=True, text=True)
    assert r.returncode == 1 and "Failed to load GGUF weights" in r.stderr


def test_reference_paged_attention_test_program_runs_against_the_library(pkg, ob, tmp_path):
    """tests/test_paged_attention.c of the C-ML tree, unmodified, builds against include/ and
    libcml_b200.so; every case that needs no device passes here (the three that call
    cml_paged_gqa_forward with valid arguments need a GPU and are covered by the GPU tests)."""
    import subprocess
    root = ob.reference_root()
    if root is None:
        pytest.skip("the C-ML source tree is not on this machine")
    exe = tmp_path / "test_paged_attention"
    libdir = ROOT / "c-ml_b200" / "lib"
    cmd = ["gcc", "-std=c11", "-D_POSIX_C_SOURCE=200809L", f"-I{ROOT / 'include'}", str(Path(root) / "tests" / "test_paged_attention.c"),
           "-o", str(exe), f"-L{libdir}", "-lcml_b200", f"-Wl,-rpath,{libdir}", "-lm"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    text = r.stdout + r.stderr
    verdicts = re.findall(r"^\s{2}(\w+)\s.*?\[(PASS|FAIL)\]", text, flags=re.M | re.S)
    failed = {name for name, v in verdicts if v == "FAIL"}
    assert len(verdicts) == 20, text[-2000:]
    assert failed <= {"paged_gqa_output_shape", "paged_gqa_multi_query_tokens", "paged_gqa_output_nonzero"}, failed


def _table_models(pkg, next_draft, next_target, vocab, fail_len):
    """ctypes callbacks of the stand-in models the golden vectors were made with (oracle/ref_driver.c:
    after token t the model predicts next[t], with an equal logit at next[t] + 1 when t is odd)."""
    keep = []

    def forward(table, fail):
        def fn(_ctx, toks, n):
            if fail and n >= fail:
                return None
            lg = np.zeros((n, vocab), np.float32)
            for r in range(n):
                nx = int(table[toks[r]])
                lg[r, nx] = 1.0
                if toks[r] & 1 and nx + 1 < vocab:
                    lg[r, nx + 1] = 1.0
            return C.cast(pkg.numpy_to_tensor(lg), C.c_void_p).value
        return pkg.ModelForwardFn(fn)

    def sample(_ctx, logits, _temperature):
        a = pkg.tensor_to_numpy(C.cast(logits, pkg.TP), free=False)
        return int(np.argmax(a[-1]))
    keep += [forward(next_draft, fail_len), forward(next_target, 0), pkg.SampleTokenFn(sample)]
    return keep


def test_speculative_decode_step_matches_the_compiled_reference(pkg, golden):
    tgt = golden["spec_target"]
    vocab = len(tgt)
    for name in ("all", "first", "mid", "giveup", "k1", "k16"):
        K, fail = (int(x) for x in golden[f"spec_{name}_cfg"])
        cfg = pkg.lib.cml_speculative_default_config()
        assert (cfg.num_draft_tokens, cfg.top_k, cfg.do_sample) == (5, 40, True) and abs(cfg.temperature - 0.8) < 1e-7
        cfg.num_draft_tokens = K
        dec = pkg.lib.cml_speculative_create(C.byref(cfg), vocab)
        assert dec
        fd, ft, fs = _table_models(pkg, golden[f"spec_{name}_draft"], tgt, vocab, fail)
        pkg.lib.cml_speculative_set_draft_model(dec, None, C.cast(fd, C.c_void_p), C.cast(fs, C.c_void_p))
        pkg.lib.cml_speculative_set_target_model(dec, None, C.cast(ft, C.c_void_p), C.cast(fs, C.c_void_p))
        prefix = np.ascontiguousarray(golden[f"spec_{name}_prefix"], np.int32)
        pkg.lib.cml_set_log_level(5)
        res = pkg.lib.cml_speculative_decode_step(dec, pkg.np_ptr(prefix), len(prefix))
        pkg.lib.cml_set_log_level(3)
        assert res
        r, want_meta, want_rates = res.contents, golden[f"spec_{name}_meta"], golden[f"spec_{name}_rates"]
        got = [r.accepted_tokens[i] for i in range(r.num_accepted)]
        assert got == golden[f"spec_{name}_tokens"][:r.num_accepted].tolist(), name
        d = dec.contents
        assert [r.num_accepted, r.num_drafted, r.num_verified, d.total_drafted, d.total_accepted, d.total_steps] == want_meta.tolist(), name
        assert r.acceptance_rate == want_rates[0] and pkg.lib.cml_speculative_acceptance_rate(dec) == want_rates[1]
        assert r.total_time_ms >= r.draft_time_ms >= 0 and r.verify_time_ms >= 0
        pkg.lib.cml_speculative_result_free(res)
        pkg.lib.cml_speculative_free(dec)


def test_speculative_argument_checks(pkg):
    pkg.lib.cml_set_log_level(5)
    cfg = pkg.lib.cml_speculative_default_config()
    assert not pkg.lib.cml_speculative_create(None, 10)
    assert not pkg.lib.cml_speculative_create(C.byref(cfg), 0)
    cfg.num_draft_tokens = 17
    assert not pkg.lib.cml_speculative_create(C.byref(cfg), 10)
    cfg.num_draft_tokens = 3
    dec = pkg.lib.cml_speculative_create(C.byref(cfg), 10)
    one = np.array([1], np.int32)
    assert not pkg.lib.cml_speculative_decode_step(dec, pkg.np_ptr(one), 1)          # callbacks not set
    assert not pkg.lib.cml_speculative_decode_step(None, pkg.np_ptr(one), 1)
    assert pkg.lib.cml_speculative_acceptance_rate(dec) == 0.0 and pkg.lib.cml_speculative_acceptance_rate(None) == 0.0
    pkg.lib.cml_speculative_free(dec)
    pkg.lib.cml_speculative_free(None)
    pkg.lib.cml_speculative_result_free(None)
    assert not pkg.lib.cml_speculative_llama_create(None, False)
    pkg.lib.cml_set_log_level(3)


def test_reference_speculative_test_program_passes_against_the_library(pkg, ob, tmp_path):
    """tests/test_speculative.c of the C-ML tree, unmodified (mock models, no device needed): 18 of 18."""
    import subprocess
    root = ob.reference_root()
    if root is None:
        pytest.skip("the C-ML source tree is not on this machine")
    exe = tmp_path / "test_speculative"
    libdir = ROOT / "c-ml_b200" / "lib"
    cmd = ["gcc", "-std=c11", "-D_POSIX_C_SOURCE=200809L", f"-I{ROOT / 'include'}", str(Path(root) / "tests" / "test_speculative.c"),
           "-o", str(exe), f"-L{libdir}", "-lcml_b200", f"-Wl,-rpath,{libdir}", "-lm"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 0 and "18/18 passed" in r.stdout, (r.stdout + r.stderr)[-1500:]


def test_reference_serving_test_program_passes_against_the_library(pkg, ob, tmp_path):
    """tests/test_serving.c of the C-ML tree, unmodified (scheduler bookkeeping only): 25 of 25."""
    import subprocess
    root = ob.reference_root()
    if root is None:
        pytest.skip("the C-ML source tree is not on this machine")
    exe = tmp_path / "test_serving"
    libdir = ROOT / "c-ml_b200" / "lib"
    cmd = ["gcc", "-std=c11", "-D_POSIX_C_SOURCE=200809L", f"-I{ROOT / 'include'}", str(Path(root) / "tests" / "test_serving.c"),
           "-o", str(exe), f"-L{libdir}", "-lcml_b200", f"-Wl,-rpath,{libdir}", "-lm"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 0 and "25/25 passed" in r.stdout, (r.stdout + r.stderr)[-1500:]
