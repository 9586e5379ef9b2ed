"""CPU checks on the C-ABI boundary: the library loads and exports every declared symbol, and
argument validation fails with the documented status before any GPU work."""
import ctypes
import re

from guffin_b200 import lib


def declared_symbols():
    text = open(lib.HEADER_PATH).read()
    return sorted(set(re.findall(r"GF_API\s+[\w\s\*]+?\b(gf_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    L = lib.load()
    names = declared_symbols()
    assert len(names) >= 20
    for name in names:
        assert hasattr(L, name), f"{name} is declared in include/guffin_b200.h but not exported"


def test_version_and_error_text():
    L = lib.load()
    assert b"sm_100a" in L.gf_version()
    assert L.gf_packed_weight_bytes(12, 100, 8) == 0          # K not a multiple of 256
    assert b"multiple" in L.gf_last_error()


def test_packed_sizes_keep_native_byte_count():
    L = lib.load()
    # 8 columns x one unit: exactly the native bytes, no padding
    assert L.gf_packed_weight_bytes(lib.Q4_K, 3840, 15360) == 15360 * 15 * 144
    assert L.gf_packed_weight_bytes(lib.Q6_K, 15360, 3840) == 3840 * 60 * 210
    assert L.gf_packed_weight_bytes(lib.Q8_0, 640, 262144) == 262144 * 20 * 34
    # a ragged last tile is zero-padded to 8 columns
    assert L.gf_packed_weight_bytes(lib.Q4_K, 256, 9) == 2304           # one group of sixteen columns
    assert L.gf_packed_weight_bytes(lib.Q4_K, 256, 17) == 2 * 2304


def test_matmul_rejects_bad_arguments_without_a_gpu():
    L = lib.load()
    assert L.gf_matmul_workspace_bytes(lib.Q4_K, 9, 3840, 15360) == 0      # rows > GF_MAX_ROWS
    assert L.gf_matmul_workspace_bytes(7, 1, 3840, 15360) == 0             # unknown dtype
    assert L.gf_matmul(lib.Q4_K, None, None, None, 0, 3840, 15360, None, None) == lib.GF_ERR_INVALID
    assert L.gf_matmul(lib.Q4_K, None, None, None, 1, 100, 15360, None, None) == lib.GF_ERR_INVALID


def test_gguf_loader_rejects_missing_arguments_without_a_gpu(tmp_path):
    L = lib.load()
    L.gf_model_load_gguf.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p]
    L.gf_model_load_gguf.restype = ctypes.c_int
    assert L.gf_model_load_gguf(None, str(tmp_path / "absent.gguf").encode(), None) == lib.GF_ERR_INVALID
    assert b"null argument" in L.gf_last_error()


def test_binding_argument_counts_match_the_header():
    """Every entry point the ctypes binding declares takes as many arguments as include/guffin_b200.h gives it (a
    binding that drifts from the header would pass garbage in the missing slots)."""
    from guffin_b200 import engine, model  # noqa: F401  (they register their signatures)
    L = lib.load()
    text = re.sub(r"/\*.*?\*/", "", open(lib.HEADER_PATH).read(), flags=re.S)
    declarations = re.findall(r"GF_API\s+[\w\s\*]+?\b(gf_\w+)\s*\(([^;]*?)\)\s*;", text, flags=re.S)
    assert len(declarations) >= 120
    checked = 0
    for name, parameters in declarations:
        parameters = parameters.strip()
        expected = 0 if parameters in ("", "void") else len(parameters.split(","))
        argtypes = getattr(L, name).argtypes
        if argtypes is None:
            assert expected == 0 or name in ("gf_last_error", "gf_version"), f"{name} has no declared argument types"
            continue
        assert len(argtypes) == expected, f"{name}: the binding passes {len(argtypes)} arguments, the header declares {expected}"
        checked += 1
    assert checked >= 110
