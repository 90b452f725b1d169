"""CPU-only: the C-ABI library loads and exports every symbol the header declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    for fn in os.listdir(os.path.join(ROOT, "include")):
        if fn.endswith(".h"):
            text = open(os.path.join(ROOT, "include", fn)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names |= set(re.findall(r"\b(wb_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_library_exports_every_declared_symbol():
    lib_path = os.path.join(ROOT, "weta_b200", "libweta_b200.so")
    assert os.path.exists(lib_path), "build the library first: python -c 'import __graft_entry__ as g; g.build()'"
    lib = ctypes.CDLL(lib_path)
    syms = declared_symbols()
    assert len(syms) > 40
    missing = [s for s in syms if not hasattr(lib, s)]
    assert not missing, f"declared in include/*.h but not exported: {missing}"


def test_no_device_means_an_error_not_a_fallback():
    from weta_b200.backend import BackendError, B200Backend, device_count
    if device_count() == 0:
        try:
            B200Backend(0)
        except BackendError as e:
            assert e.status == 5  # WB_ERR_DEVICE_UNAVAILABLE
        else:
            raise AssertionError("backend creation must fail without a GPU")


def test_host_rng_matches_the_python_statement():
    from weta_b200.backend import load_library
    from weta_b200.core import Pcg, splitmix64

    class G(ctypes.Structure):
        _fields_ = [("state", ctypes.c_uint64), ("inc", ctypes.c_uint64)]

    lib = load_library()
    lib.wb_pcg_seed.argtypes = [ctypes.POINTER(G), ctypes.c_uint64]
    lib.wb_pcg_next_u64.argtypes = [ctypes.POINTER(G)]
    lib.wb_pcg_next_u64.restype = ctypes.c_uint64
    for seed in (0, 42, 67280421310721):
        g, p = G(), Pcg(seed)
        lib.wb_pcg_seed(ctypes.byref(g), seed)
        for _ in range(8):
            assert lib.wb_pcg_next_u64(ctypes.byref(g)) == p.next_u64()
    assert lib.wb_splitmix64(42, 7) == splitmix64(42, 7)
