"""The C-ABI library loads and exports every symbol include/orangu_b200.h declares (no GPU needed)."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from orangu_b200 import build, capi

    build.build_all()
    return capi.load()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "orangu_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ob_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree(lib):
    from orangu_b200 import capi

    names = declared_symbols()
    assert len(names) >= 30
    assert set(names) == set(capi.SIGNATURES), set(names) ^ set(capi.SIGNATURES)
    for n in names:
        assert hasattr(lib, n), f"library does not export {n}"


def test_constants_without_a_device(lib):
    assert lib.ob_abi_version() == 4
    assert [lib.ob_supports_type(t) for t in (0, 8, 12, 13, 14, 2, 6, 20)] == [1, 1, 1, 1, 1, 1, 1, 1]
    assert [lib.ob_supports_type(t) for t in (1, 3, 7, 10, 11, 30)] == [0, 0, 0, 0, 0, 0]
    assert lib.ob_reduced_surface() is None


def test_init_without_a_device_is_a_status_not_a_crash(lib):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a device is present")
    h = C.c_void_p()
    rc = lib.ob_init(0, C.byref(h))
    assert rc == -3 and not h.value
    assert b"CUDA" in lib.ob_last_error(None) or lib.ob_last_error(None)
    from orangu_b200 import CudaBackend

    assert CudaBackend.try_init_index(0) is None  # Option::None, as try_init_index returns


def test_null_arguments_are_rejected(lib):
    assert lib.ob_init(0, None) == -1
    assert lib.ob_matmul(None, None, 1, None, None) == -1
    assert lib.ob_kv_len(None) == 0
    assert lib.ob_tp_unique_id(None) == -1


def test_cpp_host_wrapper_compiles():
    """include/orangu_b200.hpp (the C++ mirror of the Backend trait) must at least compile against the C header."""
    import subprocess, tempfile

    hpp = os.path.join(ROOT, "include", "orangu_b200.hpp")
    if not os.path.exists(hpp):
        pytest.skip("no C++ wrapper")
    with tempfile.TemporaryDirectory() as d:
        src = os.path.join(d, "t.cpp")
        open(src, "w").write('#include "orangu_b200.hpp"\nint main(){ return orangu::CudaBackend::try_init_index(0) ? 0 : 0; }\n')
        r = subprocess.run(["/usr/bin/g++", "-std=c++17", "-fsyntax-only", "-I", os.path.join(ROOT, "include"), src], capture_output=True, text=True)
        assert r.returncode == 0, r.stderr


def _compile_and_run(source: str, extra=(), run=True):
    import subprocess, tempfile

    from orangu_b200 import capi

    with tempfile.TemporaryDirectory() as d:
        src, exe = os.path.join(d, "t.cpp"), os.path.join(d, "t")
        open(src, "w").write(source)
        libdir = os.path.dirname(capi.lib_path())
        cmd = ["/usr/bin/g++", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"), src, "-o", exe, *extra]
        r = subprocess.run(cmd, capture_output=True, text=True)
        assert r.returncode == 0, r.stderr
        if not run:
            return ""
        r = subprocess.run([exe], capture_output=True, text=True, env={**os.environ, "LD_LIBRARY_PATH": libdir + ":" + os.environ.get("LD_LIBRARY_PATH", "")})
        assert r.returncode == 0, r.stdout + r.stderr
        return r.stdout


def test_struct_layouts_agree_between_header_binding_and_integration_notes(lib):
    """sizeof / offsetof as the C compiler sees the header == the ctypes binding == the figures INTEGRATION.md quotes for
    the Rust #[repr(C)] structs (a binding that is one field short hands the library a truncated struct)."""
    from orangu_b200 import capi

    out = _compile_and_run(
        '#include <cstdio>\n#include <cstddef>\n#include "orangu_b200.h"\n'
        'int main(){ std::printf("%zu %zu %zu %zu %zu %zu %u\\n", sizeof(ob_model_desc), sizeof(ob_layer_desc), sizeof(ob_matrix_desc),'
        ' offsetof(ob_model_desc, rope_freqs), sizeof(ob_greedy), sizeof(ob_gguf_tensor_info), OB_ABI_VERSION); }\n')
    model, layer, matrix, off_rope, greedy, tinfo, abi = (int(v) for v in out.split())
    assert (model, layer, matrix, off_rope) == (C.sizeof(capi.ModelDesc), C.sizeof(capi.LayerDesc), C.sizeof(capi.MatrixDesc), capi.ModelDesc.rope_freqs.offset)
    assert greedy == C.sizeof(capi.Greedy) and tinfo == C.sizeof(capi.GgufTensorInfo)
    assert abi == lib.ob_abi_version()
    notes = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    quoted = re.search(r"size_of::<ob_model_desc>\(\) == (\d+).*?size_of::<ob_layer_desc>\(\) == (\d+).*?OB_ABI_VERSION: u32 = (\d+)", notes, flags=re.S)
    assert quoted, "INTEGRATION.md must quote the struct sizes its Rust binding is checked against"
    assert tuple(int(v) for v in quoted.groups()) == (model, layer, abi)
    # every field of the C struct appears in the written Rust struct
    rust = notes[notes.index("pub struct ob_model_desc"):]
    rust = rust[:rust.index("}")]
    for name, _ in capi.ModelDesc._fields_:
        assert f"pub {name}:" in rust, f"INTEGRATION.md's ob_model_desc lacks {name}"
    rust_layer = notes[notes.index("pub struct ob_layer_desc"):]
    rust_layer = rust_layer[:rust_layer.index("}")]
    for name, _ in capi.LayerDesc._fields_:
        assert f"pub {name}:" in rust_layer, f"INTEGRATION.md's ob_layer_desc lacks {name}"
    header = re.sub(r"/\*.*?\*/", "", open(os.path.join(ROOT, "include", "orangu_b200.h")).read(), flags=re.S)
    for name in declared_symbols():
        assert f"pub fn {name}(" in notes, f"INTEGRATION.md does not declare {name}"
    assert header


def test_cpp_model_and_slot_pool_wrappers_compile():
    """The ModelForward / KvCache / SlotPool part of the C++ mirror, compiled with warnings on and linked against the library
    (run without a device: try_init_index gives an empty optional and main returns)."""
    src = ('#include "orangu_b200.hpp"\n'
           'int main(){ auto be = orangu::CudaBackend::try_init_index(0); if (!be) return 0; ob_model_desc d{};\n'
           ' try { orangu::LlamaModel m(*be, d); auto kv = m.new_kv_cache(16, true); auto t = m.forward_maybe_sampling(kv, {1, 2, 3}, 0);\n'
           '  (void)m.decode_greedy(kv, t); (void)m.forward(kv, {t}, kv.len()); ob_slot_pool_desc pd{2, 64, 0, 0, 0, 1}; orangu::SlotPool pool(m, pd);\n'
           '  if (auto g = pool.try_acquire(0)) { auto x = g->prefill({1, 2}); (void)g->decode(x); g->truncate(1); }\n'
           '  (void)pool.snapshot(); (void)pool.stats(); std::vector<orangu::KvCache *> c{&kv}; (void)m.forward_batch_decode(c, {1}); }\n'
           ' catch (const std::exception &) { return 0; } return 0; }\n')
    from orangu_b200 import capi

    _compile_and_run(src, extra=["-Wall", "-Wextra", "-Werror", "-L", os.path.dirname(capi.lib_path()), "-lorangu_b200"], run=False)


@pytest.mark.gpu
def test_cpp_model_and_slot_pool_run_a_gguf_model_on_the_gpu(tmp_path):
    """A tiny model written to a .gguf file, opened by the library, run through the C++ classes: prefill + greedy decode through
    LlamaModel (reserved and paged caches) and through a SlotPool guard give the oracle's tokens."""
    import numpy as np

    import oracle as O
    from orangu_b200 import capi, synth
    from orangu_b200.gguf import write_gguf

    cfg = dict(synth.CONFIGS["tiny"])
    tensors = synth.model_tensors(cfg, seed=31)
    path = str(tmp_path / "tiny.gguf")
    write_gguf(path, cfg, tensors)
    toks = np.random.default_rng(3).integers(0, cfg["n_vocab"], 21).astype(np.uint32)
    ref = O.Model(cfg, tensors)
    rkv = ref.new_kv(64, f16=True)
    want = [O.argmax(ref.forward(rkv, toks, 0))]
    for i in range(5):
        want.append(O.argmax(ref.forward(rkv, [want[-1]], 21 + i)))
    src = (
        '#include <cstdio>\n#include "orangu_b200.hpp"\n'
        'int main(){ auto be = orangu::CudaBackend::try_init_index(0); if (!be) return 3;\n'
        ' ob_gguf *g = nullptr; if (ob_gguf_open("%s", &g) != OB_OK) return 4; ob_model_desc d{}; if (ob_gguf_model_desc(g, &d) != OB_OK) return 5;\n'
        ' d.max_seq_len = 64; d.max_batch_tokens = 16; orangu::LlamaModel m(*be, d); ob_gguf_close(g);\n'
        ' std::vector<uint32_t> toks{%s};\n'
        ' for (int paged = 0; paged < 2; ++paged) { auto kv = m.new_kv_cache(48, paged != 0); uint32_t t = m.forward_maybe_sampling(kv, toks, 0); std::printf("%%u", t);\n'
        '  for (int i = 0; i < 5; ++i) { t = i %% 2 ? m.decode_greedy(kv, t) : m.forward_maybe_sampling(kv, {t}, kv.len()); std::printf(" %%u", t); } std::printf("\\n"); }\n'
        ' ob_slot_pool_desc pd{2, 48, 0, 1, 8, 1}; orangu::SlotPool pool(m, pd); auto s = pool.try_acquire(0); if (!s) return 6;\n'
        ' uint32_t t = s->prefill(toks); std::printf("%%u", t); for (int i = 0; i < 5; ++i) { t = s->decode(t); std::printf(" %%u", t); } std::printf("\\n");\n'
        ' return pool.stats().busy == 1 ? 0 : 7; }\n' % (path, ", ".join(str(int(t)) for t in toks)))
    out = _compile_and_run(src, extra=["-L", os.path.dirname(capi.lib_path()), "-lorangu_b200"])
    lines = [[int(v) for v in ln.split()] for ln in out.strip().splitlines()]
    assert lines == [want, want, want], (lines, want)


def test_row_bytes_of_the_cpp_wrapper_for_every_type():
    out = _compile_and_run(
        '#include <cstdio>\n#include "orangu_b200.hpp"\n'
        'int main(){ for (unsigned t : {8u, 12u, 13u, 14u, 2u, 6u, 20u}) { orangu::QuantMatrix m{nullptr, t, 4096, 3}; std::printf("%llu ", (unsigned long long)m.row_bytes()); } }\n',
        extra=["-L", os.path.dirname(__import__("orangu_b200").capi.lib_path()), "-lorangu_b200"])
    assert [int(v) for v in out.split()] == [4096 // 32 * 34, 4096 // 256 * 144, 4096 // 256 * 176, 4096 // 256 * 210, 4096 // 32 * 18, 4096 // 32 * 22, 4096 // 32 * 18]


@pytest.mark.gpu
def test_cpp_host_wrapper_runs_a_matmul_on_the_gpu():
    """The C++ mirror of the Backend trait, compiled and run: one Q4_0 and one Q4_K product through the class equal the
    oracle's (the Q4_0 row size is what the wrapper once got wrong)."""
    import numpy as np

    import oracle as O
    from orangu_b200 import capi, synth

    out_dim, in_dim = 6, 512
    cases = []
    with __import__("tempfile").TemporaryDirectory() as d:
        for t in (2, 12):
            raw = synth.matrix(t, out_dim, in_dim, 5 + t)["data"]
            x = synth.normal(in_dim, 9 + t)
            raw.tofile(os.path.join(d, f"w{t}.bin"))
            x.tofile(os.path.join(d, f"x{t}.bin"))
            cases.append((t, raw, x))
        src = (
            '#include <cstdio>\n#include <vector>\n#include <fstream>\n#include <iterator>\n#include "orangu_b200.hpp"\n'
            'static std::vector<char> rd(const std::string &p){ std::ifstream f(p, std::ios::binary); return {std::istreambuf_iterator<char>(f), {}}; }\n'
            'int main(int, char **argv){ std::string d = "%s"; auto be = orangu::CudaBackend::try_init_index(0); if (!be) return 3;\n'
            ' for (unsigned t : {2u, 12u}) { auto w = rd(d + "/w" + std::to_string(t) + ".bin"); auto x = rd(d + "/x" + std::to_string(t) + ".bin");\n'
            '  orangu::QuantMatrix m{reinterpret_cast<const uint8_t *>(w.data()), t, %du, %du}; if (m.row_bytes() * m.out_dim != w.size()) return 4;\n'
            '  auto y = be->matmul(reinterpret_cast<const float *>(x.data()), 1, m); std::ofstream o(d + "/y" + std::to_string(t) + ".bin", std::ios::binary);\n'
            '  o.write(reinterpret_cast<const char *>(y.data()), y.size() * 4); }\n return 0; }\n' % (d, in_dim, out_dim))
        _compile_and_run(src, extra=["-L", os.path.dirname(capi.lib_path()), "-lorangu_b200"])
        for t, raw, x in cases:
            got = np.fromfile(os.path.join(d, f"y{t}.bin"), dtype=np.float32)
            want = O.matmul(x, 1, raw, t, in_dim, out_dim)
            assert (got.view(np.uint32) == want.view(np.uint32)).all()
