"""The C-ABI library without a GPU: it loads, exports every function that
include/h3q8.h declares (in the spirit of h3cli's tests/test_gpu_contract.c and
tests/check_gpu_contract.py), its host packer reproduces the reference's golden
vectors, and the GPU operators refuse to run instead of falling back."""
import ctypes
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")


@pytest.fixture(scope="module")
def lib():
    from h3cli_b200 import build
    build.build()
    import h3cli_b200
    return h3cli_b200.library()


def declared_functions():
    text = open(os.path.join(ROOT, "include", "h3q8.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"typedef\s+(struct|enum)\s*\{.*?\}\s*\w+\s*;", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(h3q?8?_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(lib):
    names = declared_functions()
    assert len(names) >= 60
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/h3q8.h but not exported"
        assert name in lib._signatures, f"{name} has no ctypes signature in h3cli_b200/api.py"
    assert set(lib._signatures) <= set(names), "the binding names a function the header does not declare"


def test_host_packer_known_answers(lib):
    # tests/metal_q8.c:21-34 through the library's own h3_q8_* symbols
    g = np.load(os.path.join(GOLDEN, "q8_pack.npz"))
    src = np.ascontiguousarray(g["known_src"])
    q = np.empty((1, 65), np.int8)
    s = np.empty((1, 2), np.float32)
    assert lib.h3_q8_pack_rows(src.ctypes.data, q.ctypes.data, s.ctypes.data, 1, 65)
    assert q[0, :8].tolist() == [127, -127, 0, 2, 2, 0, -2, -2] and (s == 1).all() and q[0, 64] == 0
    off, total = ctypes.c_size_t(), ctypes.c_size_t()
    assert lib.h3_q8_layout(1, 65, ctypes.byref(off), ctypes.byref(total)) and (off.value, total.value) == (68, 76)
    assert not lib.h3_q8_layout(0, 65, ctypes.byref(off), ctypes.byref(total))
    assert not lib.h3_q8_layout(0xFFFFFFFF, 0xFFFFFFFF, ctypes.byref(off), ctypes.byref(total))
    assert not lib.h3_q8_layout(1, 0xFFFFFFFF - 31, ctypes.byref(off), ctypes.byref(total))
    for bad in (0x7FC0, 0x7F80):
        src[0, 64] = bad
        assert not lib.h3_q8_pack_rows(src.ctypes.data, q.ctypes.data, s.ctypes.data, 1, 65)
    src[0, 64] = 1
    assert lib.h3_q8_pack_rows(src.ctypes.data, q.ctypes.data, s.ctypes.data, 1, 65) and np.isfinite(s).all()


def test_host_packer_matches_reference_fixtures(lib, oracle):
    g = np.load(os.path.join(GOLDEN, "q8_pack.npz"))
    for i in range(4):
        src = np.ascontiguousarray(g[f"src{i}"])
        rows, cols = src.shape
        q = np.empty((rows, cols), np.int8)
        s = np.empty(g[f"s{i}"].shape, np.float32)
        assert lib.h3_q8_pack_rows(src.ctypes.data, q.ctypes.data, s.ctypes.data, rows, cols)
        assert (q == g[f"q{i}"]).all() and (s.view(np.uint32) == g[f"s{i}"].view(np.uint32)).all()
    rng = np.random.default_rng(3)
    w = oracle.f32_to_bf16(rng.standard_normal((12, 400)).astype(np.float32)).reshape(12, 400)
    for group in (0, 64, 128):
        want_q, want_s = oracle.q8_pack_rows(w, group)
        q = np.empty_like(want_q)
        s = np.empty_like(want_s)
        assert lib.h3q8_q8_pack_rows(w.ctypes.data, q.ctypes.data, s.ctypes.data, 12, 400, group)
        assert (q == want_q).all() and (s.view(np.uint32) == want_s.view(np.uint32)).all()


def test_no_cpu_fallback(lib):
    import h3cli_b200
    buf = ctypes.create_string_buffer(256)
    handle = lib.h3_gpu_create(b"", buf, len(buf))
    if handle:  # a GPU is present: nothing to refuse
        lib.h3_gpu_free(handle)
        pytest.skip("a CUDA device is present")
    assert b"no CPU path" in buf.value or b"sm_100a" in buf.value
    with pytest.raises(h3cli_b200.H3Error):
        h3cli_b200.Gpu()
    d = h3cli_b200.LinearDesc(mode=1, rows=4, input_dim=16, output_dim=8)
    assert lib.h3q8_linear(ctypes.byref(d), None) == 0 and lib.h3q8_last_error()


# --------------------------------------------------------------------------- drop-in checks against the reference's headers
REF_BUILD = os.path.join(ROOT, "oracle", "_ref")


def reference_tree():
    import oracle
    return oracle._reference_tree()


def test_stats_layout_equals_the_reference_struct(lib, tmp_path):
    """h3_gpu_stats as include/h3q8.h declares it, as ctypes mirrors it and as the reference's src/gpu.h:99-142
    lays it out (oracle/_ref/abi_layout_reference.txt, written by tests/abi/contract.c compiled against that
    header): same size, same offset for every counter this path feeds."""
    import subprocess
    import h3cli_b200
    binary = tmp_path / "layout_mine"
    subprocess.run(["gcc", "-std=c11", "-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "abi", "layout_mine.c"),
                    "-o", str(binary)], check=True)
    mine = subprocess.run([str(binary)], check=True, capture_output=True, text=True).stdout
    fields = dict(line.split() for line in mine.splitlines())
    assert int(fields.pop("sizeof")) == ctypes.sizeof(h3cli_b200.api.Stats)
    for name, offset in fields.items():
        assert getattr(h3cli_b200.api.Stats, name).offset == int(offset), name
    reference = os.path.join(REF_BUILD, "abi_layout_reference.txt")
    if not os.path.exists(reference):
        pytest.skip("oracle/_ref was built without the reference tree")
    assert open(reference).read() == mine


def test_contract_binary_links_every_symbol_through_the_reference_header():
    """tests/abi/contract.c includes only the reference's headers and links libh3q8: every symbol of the path resolves."""
    import subprocess
    binary = os.path.join(REF_BUILD, "abi_contract")
    if not os.path.exists(binary):
        pytest.skip("oracle/_ref/abi_contract was not built (no reference tree at build time)")
    out = subprocess.run([binary], check=True, capture_output=True, text=True).stdout
    assert int(out.split()[0]) >= 60


def prototypes(text, wanted=None):
    """name -> normalised 'return type | parameter types' of every function declared in a C header."""
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    text = re.sub(r"//[^\n]*", " ", text)
    text = re.sub(r"#[^\n]*", " ", text)
    found = {}
    for match in re.finditer(r"([A-Za-z_][A-Za-z0-9_ \t\n\*]*?)\b(h3_[a-z0-9_]+)\s*\(([^;{}]*?)\)\s*;", text):
        ret, name, params = match.groups()
        if wanted is not None and name not in wanted:
            continue
        def kind(p):
            p = re.sub(r"\s+", " ", p.strip())
            p = re.sub(r"\b[a-z_][a-z0-9_]*$", "", p) if not p.endswith("*") and " " in p else p   # drop the parameter name
            return re.sub(r"\s*\*\s*", "*", p).strip()
        found[name] = (re.sub(r"\s+", " ", ret.strip()), [kind(p) for p in params.split(",")])
    return found


def test_prototypes_equal_the_reference_headers():
    """Every h3_* function this header shares with src/gpu.h / src/weights/residency.h / src/weights/q8.h has the
    reference's return type and parameter types (names may differ).  Needs the reference tree; skipped without it."""
    tree = reference_tree()
    if not tree:
        pytest.skip("reference tree not present")
    mine = prototypes(open(os.path.join(ROOT, "include", "h3q8.h")).read())
    theirs = {}
    for header in ("src/gpu.h", "src/weights/residency.h", "src/weights/q8.h", "src/weights/quant.h"):
        theirs.update(prototypes(open(os.path.join(tree, header)).read()))
    shared = sorted(set(mine) & set(theirs))
    assert len(shared) >= 55
    for name in shared:
        assert mine[name] == theirs[name], f"{name}: {mine[name]} != reference {theirs[name]}"
