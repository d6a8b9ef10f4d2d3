"""The packed-weight artifact cache on the host (no GPU), in the manner of h3cli's
tests/test_quant_cache.c: key stability under path aliases, key separation by offset /
shape / group, rejection of truncated, corrupted and bit-flipped artifacts (an error, not a
miss), source mutation, and concurrent writers."""
import ctypes
import multiprocessing
import os

import numpy as np
import pytest

ROWS, COLS, GROUP = 128, 256, 64


@pytest.fixture(scope="module")
def lib():
    from h3cli_b200 import build
    build.build()
    import h3cli_b200
    return h3cli_b200.library()


def open_entry(lib, directory, source, offset=0, rows=ROWS, cols=COLS, group=GROUP):
    error = ctypes.create_string_buffer(512)
    entry = lib.h3q8_cache_open(str(directory).encode(), str(source).encode(), offset, rows, cols, group, error, len(error))
    return entry, error.value.decode()


def make_source(path, matrices=2, seed=0):
    data = np.random.default_rng(seed).integers(0, 65535, matrices * ROWS * COLS, dtype=np.uint16)
    path.write_bytes(data.tobytes())
    return path


def test_roundtrip_and_key_rules(lib, tmp_path):
    source = make_source(tmp_path / "weights.bin")
    cache = tmp_path / "cache"
    cache.mkdir()
    entry, why = open_entry(lib, cache, source)
    assert entry, why
    size = lib.h3q8_cache_payload_bytes(entry)
    offset = ctypes.c_size_t()
    assert size == lib.h3q8_q8_blob_bytes(ROWS, COLS, GROUP, ctypes.byref(offset)) and size % 256 == 0
    payload = np.random.default_rng(1).integers(0, 255, size, dtype=np.uint8)
    back = np.zeros(size, np.uint8)
    error = ctypes.create_string_buffer(512)
    assert lib.h3q8_cache_read(entry, back.ctypes.data, error, len(error)) == 0            # absent
    assert lib.h3q8_cache_write(entry, payload.ctypes.data, error, len(error)) == 1
    assert lib.h3q8_cache_read(entry, back.ctypes.data, error, len(error)) == 1 and (back == payload).all()
    artifact = lib.h3q8_cache_artifact(entry).decode()
    lib.h3q8_cache_close(entry)
    assert os.path.exists(artifact) and not [f for f in os.listdir(cache) if ".tmp." in f]
    # the same file through a symlink and a relative path is the same artifact
    link = tmp_path / "alias.bin"
    link.symlink_to(source)
    for alias in (link, tmp_path / "." / "weights.bin"):
        entry, why = open_entry(lib, cache, alias)
        assert entry, why
        assert lib.h3q8_cache_artifact(entry).decode() == artifact
        lib.h3q8_cache_close(entry)
    # offset, shape and group each select another artifact
    for kwargs in (dict(offset=ROWS * COLS * 2), dict(rows=64), dict(cols=128), dict(group=128), dict(group=0)):
        entry, why = open_entry(lib, cache, source, **kwargs)
        assert entry, why
        assert lib.h3q8_cache_artifact(entry).decode() != artifact
        lib.h3q8_cache_close(entry)
    # invalid requests
    for kwargs in (dict(offset=1), dict(offset=3 * ROWS * COLS * 2), dict(rows=0), dict(rows=ROWS * 3)):
        entry, why = open_entry(lib, cache, source, **kwargs)
        assert not entry and why
    assert not open_entry(lib, cache, tmp_path / "missing.bin")[0]


def test_damaged_artifacts_are_errors_not_misses(lib, tmp_path):
    source = make_source(tmp_path / "weights.bin")
    cache = tmp_path / "cache"
    cache.mkdir()
    entry, _ = open_entry(lib, cache, source)
    size = lib.h3q8_cache_payload_bytes(entry)
    payload = np.arange(size, dtype=np.uint64).astype(np.uint8)
    error = ctypes.create_string_buffer(512)
    assert lib.h3q8_cache_write(entry, payload.ctypes.data, error, len(error))
    artifact = lib.h3q8_cache_artifact(entry).decode()
    good = open(artifact, "rb").read()
    back = np.zeros(size, np.uint8)
    for damaged in (good[:-1], good[:64], good + b"x", bytes([good[0] ^ 1]) + good[1:], good[:20] + bytes([good[20] ^ 4]) + good[21:],
                    good[:60] + bytes([good[60] ^ 0x80]) + good[61:]):
        open(artifact, "wb").write(damaged)
        assert lib.h3q8_cache_read(entry, back.ctypes.data, error, len(error)) == -1
        assert b"corrupt" in error.value
    open(artifact, "wb").write(good)
    assert lib.h3q8_cache_read(entry, back.ctypes.data, error, len(error)) == 1
    # payload corruption is outside what a metadata cache can see (the reference's is the same); header is what is checked
    # source mutation: the open entry notices, and a new open keys a new artifact
    os.utime(source, ns=(1, 1))
    assert lib.h3q8_cache_unchanged(entry, error, len(error)) == 0
    assert lib.h3q8_cache_read(entry, back.ctypes.data, error, len(error)) == -1
    assert lib.h3q8_cache_write(entry, payload.ctypes.data, error, len(error)) == 0
    lib.h3q8_cache_close(entry)
    entry, why = open_entry(lib, cache, source)
    assert entry and lib.h3q8_cache_artifact(entry).decode() != artifact
    assert lib.h3q8_cache_read(entry, back.ctypes.data, error, len(error)) == 0
    lib.h3q8_cache_close(entry)


def _writer(args):
    directory, source, seed = args
    import h3cli_b200
    lib = h3cli_b200.library()
    error = ctypes.create_string_buffer(512)
    entry = lib.h3q8_cache_open(directory.encode(), source.encode(), 0, ROWS, COLS, GROUP, error, len(error))
    if not entry:
        return "open failed: " + error.value.decode()
    size = lib.h3q8_cache_payload_bytes(entry)
    back = np.zeros(size, np.uint8)
    status = lib.h3q8_cache_read(entry, back.ctypes.data, error, len(error))
    if status == 0:  # holder of the lock prepares; everyone else then hits
        payload = np.full(size, 7, np.uint8)
        if not lib.h3q8_cache_write(entry, payload.ctypes.data, error, len(error)):
            status = -1
    elif status == 1 and not (back == 7).all():
        status = -1
    lib.h3q8_cache_close(entry)
    return status


def test_concurrent_preparers_publish_once(lib, tmp_path):
    source = make_source(tmp_path / "weights.bin")
    cache = tmp_path / "cache"
    cache.mkdir()
    with multiprocessing.get_context("spawn").Pool(4) as pool:
        results = pool.map(_writer, [(str(cache), str(source), i) for i in range(8)])
    assert sorted(results) == [0] + [1] * 7, results       # one preparation, seven hits, no torn reads
    assert len([f for f in os.listdir(cache) if f.endswith(".h3q8")]) == 1


def test_sha256_known_answers(lib):
    """FIPS 180-4 vectors and agreement with hashlib across block boundaries."""
    import hashlib
    out = ctypes.create_string_buffer(32)
    for message in (b"", b"abc", b"abcdbcdecdefdefgefghfghighijhijkijkljklmklmnlmnomnopnopq", b"a" * 55, b"a" * 56, b"a" * 63, b"a" * 64,
                    b"a" * 65, b"a" * 119, b"a" * 120, bytes(range(256)) * 1000):
        lib.h3q8_sha256(message, len(message), out)
        assert out.raw == hashlib.sha256(message).digest(), len(message)
    lib.h3q8_sha256(b"abc", 3, out)
    assert out.raw.hex() == "ba7816bf8f01cfea414140de5dae2223b00361a396177a9cb410ff61f20015ad"


def test_two_sources_never_validate_each_others_artifact(lib, tmp_path):
    """Different files of the same shape (paths that differ in one character, equal sizes) get different keys, and an
    artifact copied under the other key's name is refused because the key is also inside the header."""
    cache = tmp_path / "cache"
    cache.mkdir()
    a, b = make_source(tmp_path / "weights-a.bin", seed=1), make_source(tmp_path / "weights-b.bin", seed=2)
    error = ctypes.create_string_buffer(512)
    entry_a, _ = open_entry(lib, cache, a)
    entry_b, _ = open_entry(lib, cache, b)
    path_a, path_b = lib.h3q8_cache_artifact(entry_a).decode(), lib.h3q8_cache_artifact(entry_b).decode()
    assert path_a != path_b
    size = lib.h3q8_cache_payload_bytes(entry_a)
    payload, back = np.full(size, 3, np.uint8), np.zeros(size, np.uint8)
    assert lib.h3q8_cache_write(entry_a, payload.ctypes.data, error, len(error))
    open(path_b, "wb").write(open(path_a, "rb").read())                 # a's artifact under b's name
    assert lib.h3q8_cache_read(entry_b, back.ctypes.data, error, len(error)) == -1 and b"corrupt or incompatible" in error.value
    lib.h3q8_cache_close(entry_a)
    lib.h3q8_cache_close(entry_b)


def test_content_keyed_artifacts(lib, tmp_path):
    """The strict kind (src/cuda/cuda_quant.cuh:186-256): keyed by the matrix bytes, so the same weights under another
    path or at another offset are the same artifact, different weights are another one, and a flipped payload bit is
    caught by the payload digest."""
    cache = tmp_path / "cache"
    cache.mkdir()
    source = make_source(tmp_path / "weights.bin", matrices=2, seed=5)
    matrix = ROWS * COLS * 2
    data = source.read_bytes()
    copy = tmp_path / "elsewhere.bin"
    copy.write_bytes(b"\0" * 64 + data[:matrix])                       # same first matrix at offset 64 of another file

    def open_content(path, offset):
        error = ctypes.create_string_buffer(512)
        entry = lib.h3q8_cache_open_content(str(cache).encode(), str(path).encode(), offset, ROWS, COLS, GROUP, error, len(error))
        assert entry, error.value
        return entry

    # an open entry holds its artifact's lock, so entries of the SAME artifact are opened one after the other
    first, other = open_content(source, 0), open_content(source, matrix)
    name = lambda e: lib.h3q8_cache_artifact(e).decode()
    first_name = name(first)
    assert first_name != name(other) and "content" in first_name
    error = ctypes.create_string_buffer(512)
    size = lib.h3q8_cache_payload_bytes(first)
    payload, back = np.random.default_rng(9).integers(0, 255, size, dtype=np.uint8), np.zeros(size, np.uint8)
    assert lib.h3q8_cache_read(first, back.ctypes.data, error, len(error)) == 0
    assert lib.h3q8_cache_write(first, payload.ctypes.data, error, len(error))
    lib.h3q8_cache_close(first)
    same = open_content(copy, 64)
    assert name(same) == first_name
    assert lib.h3q8_cache_read(same, back.ctypes.data, error, len(error)) == 1 and (back == payload).all()
    assert lib.h3q8_cache_read(other, back.ctypes.data, error, len(error)) == 0
    good = open(name(same), "rb").read()
    flipped = bytearray(good)
    flipped[128 + size // 2] ^= 1                                           # one payload bit
    open(name(same), "wb").write(bytes(flipped))
    assert lib.h3q8_cache_read(same, back.ctypes.data, error, len(error)) == -1 and b"corrupt" in error.value
    open(name(same), "wb").write(good)
    assert lib.h3q8_cache_read(same, back.ctypes.data, error, len(error)) == 1
    lib.h3q8_cache_close(same)
    lib.h3q8_cache_close(other)
