"""h3q8_prepare's safetensors scan, without a GPU (listing mode)."""
import os
import subprocess

import numpy as np

from h3cli_b200 import build
from safetensors_fixture import write_directory


def tool():
    build.build()
    return build.PREPARE


def test_listing_finds_every_projection(tmp_path):
    written = write_directory(tmp_path)
    out = subprocess.run([tool(), "list", str(tmp_path)], check=True, capture_output=True, text=True).stdout.split("\n")
    listed = {}
    for line in filter(None, out):
        name, rows, cols, offset = line.split()
        listed[name] = (int(rows), int(cols), int(offset))
    assert set(listed) == set(written) and len(listed) == 8
    for name, (path, offset, w) in written.items():
        assert listed[name] == (w.shape[0], w.shape[1], offset)
        with open(path, "rb") as f:
            f.seek(offset)
            assert (np.frombuffer(f.read(w.nbytes), dtype=np.uint16).reshape(w.shape) == w).all()


def test_malformed_directories_are_refused(tmp_path):
    empty = tmp_path / "empty"
    empty.mkdir()
    assert subprocess.run([tool(), "list", str(empty)], capture_output=True).returncode == 1
    bad = tmp_path / "bad"
    bad.mkdir()
    (bad / "model.safetensors").write_bytes((40).to_bytes(8, "little") + b'{"blocks.0.mlp.fc1.weight": {"dtype": "BF')
    r = subprocess.run([tool(), "list", str(bad)], capture_output=True, text=True)
    assert r.returncode == 1 and "safetensors header" in r.stderr
    wrong = tmp_path / "wrong"
    wrong.mkdir()
    header = b'{"blocks.0.mlp.fc1.weight":{"dtype":"F16","shape":[128,128],"data_offsets":[0,32768]}}'
    (wrong / "model.safetensors").write_bytes(len(header).to_bytes(8, "little") + header + bytes(32768))
    r = subprocess.run([tool(), "list", str(wrong)], capture_output=True, text=True)
    assert r.returncode == 1 and "missing/invalid blocks.0.mlp.fc1.weight" in r.stderr
    assert subprocess.run([tool(), "fp8", str(wrong), str(tmp_path)], capture_output=True).returncode == 2
