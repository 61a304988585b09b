"""CPU checks of the C-ABI boundary: the library builds, loads without a GPU, and exports
exactly what include/maize_gemm.h declares.  No compute call is made here."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "maize_gemm.h"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"MAIZE_API[^;(]*?\b(maize_[a-z0-9_]+)\s*\(", text)))


def test_header_lists_entry_points():
    names = declared_symbols()
    for must in ("maize_gemm_bf16", "maize_gemm_bf16_m", "maize_gemm_bf16_ld", "maize_gemm_bf16_host",
                 "maize_ctx_create", "maize_ctx_destroy", "maize_ctx_poll"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from maize_b200 import _ffi, build
    build.build()
    lib = ctypes.CDLL(str(_ffi.LIB_PATH))
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in maize_gemm.h but not exported"


def test_binding_covers_the_header():
    from maize_b200 import _ffi
    assert sorted(_ffi.SYMBOLS) == declared_symbols()
    _ffi.load()


def test_header_compiles_as_plain_c(tmp_path):
    import subprocess
    src = tmp_path / "t.c"
    src.write_text('#include "maize_gemm.h"\n'
                   "_Static_assert(sizeof(maize_global_matrix_t) == 16, \"16-byte bundle\");\n"
                   "_Static_assert(_Alignof(maize_global_matrix_t) == 16, \"16-byte aligned\");\n"
                   "int main(void) { return MAIZE_OK; }\n")
    subprocess.run(["gcc", "-std=c11", "-Wall", "-Werror", "-I", str(ROOT / "include"), "-c", str(src), "-o",
                    str(tmp_path / "t.o")], check=True)


def test_status_strings_and_kernel_table():
    from maize_b200 import _ffi
    lib = _ffi.load()
    assert lib.maize_version() >= 100
    for code in range(7):
        assert lib.maize_status_string(code)
    names = []
    i = 1
    while lib.maize_kernel_name(i):
        names.append(lib.maize_kernel_name(i).decode())
        i += 1
    assert names and all(n.startswith("sm100_") for n in names)
    assert lib.maize_kernel_name(0) is None


def test_no_device_is_reported_not_hidden():
    """Without a GPU the context constructor fails with NO_DEVICE: there is no CPU path to fall back to."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import maize_b200
    with pytest.raises(maize_b200.MaizeError) as e:
        maize_b200.Context(0)
    assert e.value.status == maize_b200._ffi.NO_DEVICE


def test_null_context_is_rejected():
    from maize_b200 import _ffi
    lib = _ffi.load()
    assert lib.maize_gemm_bf16(None, None, 1, 8, None, 1, 8, None, 1, 1, None) == _ffi.INVALID_ARG
    assert lib.maize_ctx_poll(None, None) == _ffi.INVALID_ARG
    assert lib.maize_ctx_create(0, None) == _ffi.INVALID_ARG


def test_tile_descriptors_keep_reference_names():
    from maize_b200.tile import DType, Shape, Stride, Tile
    assert DType.from_str("F32") is DType.F32 and DType.try_from_str("nope") is None
    with pytest.raises(ValueError):
        DType.from_str("F16")
    s = Shape(128, Shape(8, 8))
    assert s.size() == 8192 and repr(s) == "(128, (8, 8))" and s == Shape(128, Shape(8, 8))
    assert Stride(64, 1) != Shape(64, 1)
    t = Tile(Shape(128, 64), DType.BF16)
    assert repr(t) == "Tile(shape=(128, 64), dtype=BF16)" and t.nbytes() == 16384
    with pytest.raises(TypeError):
        Tile((128, 64), DType.BF16)


def test_kernel_selection_table():
    """The shape -> kernel heuristic, asked without a context (148 SMs assumed): 256-wide tiles whenever N allows,
    pair or single CTA by whole waves, narrow tiles only for narrow N, the decode kernels for M <= 128."""
    from maize_b200 import _ffi
    lib = _ffi.load()

    def pick(m, n, k):
        return lib.maize_kernel_name(lib.maize_pick_kernel(None, m, n, k)).decode()

    assert pick(16384, 16384, 16384) == "sm100_2cta_256x256x128_s3"
    assert pick(4096, 4096, 4096) == "sm100_2cta_256x256x128_s3"
    assert pick(4111, 3967, 4104) == "sm100_2cta_256x256x128_s3"
    assert pick(2304, 2048, 16384) == "sm100_2cta_256x256x128_s3"   # one wave either way: the pair wins ties
    assert pick(384, 19000, 4096) == "sm100_1cta_128x256x64_s4"     # 225 single tiles: 2 waves; 150 pair tiles: 3
    assert pick(4096, 128, 4096) == "sm100_1cta_128x128x64_s6"
    assert pick(4096, 64, 4096) == "sm100_1cta_128x64x64_s8"
    assert pick(4096, 24, 4096) == "sm100_1cta_128x32x64_s8"
    assert pick(16, 16384, 4096) == "sm100_skinny_pair_m32_128xNx64_s4"
    assert pick(16, 300000, 64) == "sm100_skinny_m32_128x256x64_s4"  # more than one wave of pairs: stream-K
    assert pick(100, 4096, 4096) == "sm100_skinny_pair_m128_128xNx64_s4"  # one wave of pairs covers N
    assert pick(100, 40000, 512) == "sm100_skinny_m128_128x256x64_s4"     # it does not: stream-K


def _split_args(arglist):
    """Top-level comma split of a parameter list (no nested parentheses in this API)."""
    args = [a.strip() for a in arglist.split(",")]
    return [a for a in args if a and a != "void"]


def test_rust_binding_in_the_integration_notes_matches_the_header():
    """The extern "C" block a maintainer of the reference would add cannot be compiled here (no Rust toolchain),
    so its function names, argument counts and pointer/integer kinds are checked against the header as text."""
    notes = (ROOT / "INTEGRATION.md").read_text()
    block = re.search(r"```rust(.*?)```", notes, flags=re.S).group(1)
    block = re.sub(r"//[^\n]*", "", block)
    extern = re.search(r'extern "C" \{(.*?)\n\}', block, flags=re.S).group(1)
    rust = {name: _split_args(args) for name, args in re.findall(r"pub fn (maize_[a-z0-9_]+)\((.*?)\)", extern, flags=re.S)}
    assert len(rust) >= 8
    header = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    for name, rust_args in rust.items():
        m = re.search(r"MAIZE_API[^;(]*?\b" + name + r"\s*\((.*?)\)\s*;", header, flags=re.S)
        assert m, f"{name} is bound in the Rust block but not declared in the header"
        c_args = _split_args(m.group(1))
        assert len(c_args) == len(rust_args), (name, c_args, rust_args)
        for c_arg, r_arg in zip(c_args, rust_args):
            r_type = r_arg.split(":", 1)[1].strip()
            assert ("*" in c_arg) == r_type.startswith("*"), (name, c_arg, r_arg)
            if "*" not in c_arg:
                width = {"uint32_t": "u32", "uint64_t": "u64", "int": "c_int", "int64_t": "i64"}[c_arg.split()[0]]
                assert r_type == width, (name, c_arg, r_arg)


def test_every_tunable_is_documented_in_the_header():
    """Every key that maize_ctx_set / maize_ctx_get / maize_mgpu_set accept appears, quoted, in the header's text."""
    root = Path(__file__).resolve().parent.parent
    header = (root / "include" / "maize_gemm.h").read_text()
    keys = set()
    for name in ("maize_gemm.cu", "maize_mgpu.cu"):
        src = (root / "maize_b200" / "csrc" / name).read_text()
        keys |= set(re.findall(r'strcmp\(key, "([a-z_0-9]+)"\)', src))
    assert len(keys) >= 20
    missing = sorted(k for k in keys if f'"{k}"' not in header)
    assert not missing, missing
