"""Writes a small synthetic transformer directory in the safetensors layout (u64 header length,
JSON header, payload) for the preparation-tool tests."""
import json
import struct

import numpy as np

from h3cli_b200 import synth

PROJECTIONS = ("attn.qkv_proj.weight", "attn.out_proj.weight", "mlp.fc1.weight", "mlp.fc2.weight")


def write_directory(directory, blocks=2, hidden=128, ffn=256):
    """Two shard files; returns {name: (path, byte offset, bf16 bits [rows, cols])}."""
    shapes = {PROJECTIONS[0]: (3 * hidden, hidden), PROJECTIONS[1]: (hidden, hidden), PROJECTIONS[2]: (ffn, hidden),
              PROJECTIONS[3]: (hidden, ffn)}
    written = {}
    for shard in range(2):
        entries, payload, cursor = {"__metadata__": {"format": "pt", "note": 'a "quoted" value, [brackets] {braces}'}}, [], 0
        names = [(b, p) for b in range(blocks) for p in PROJECTIONS if (b + PROJECTIONS.index(p)) % 2 == shard]
        extra = np.arange(6, dtype=np.float32)            # a tensor the tool must skip
        entries["blocks.0.norm.scale"] = {"dtype": "F32", "shape": [6], "data_offsets": [0, 24]}
        payload.append(extra.tobytes())
        cursor = 24
        local = []
        for block, projection in names:
            rows, cols = shapes[projection]
            w = synth.bf16_normal(500 + block, PROJECTIONS.index(projection), rows, cols, 0, 0.05).reshape(rows, cols)
            name = f"blocks.{block}.{projection}"
            entries[name] = {"dtype": "BF16", "shape": [rows, cols], "data_offsets": [cursor, cursor + w.nbytes]}
            local.append((name, cursor, w))
            payload.append(w.tobytes())
            cursor += w.nbytes
        header = json.dumps(entries, indent=1 if shard else None).encode()
        header += b" " * (-len(header) % 8)
        path = directory / f"diffusion_pytorch_model-{shard + 1:05d}-of-00002.safetensors"
        path.write_bytes(struct.pack("<Q", len(header)) + header + b"".join(payload))
        for name, offset, w in local:
            written[name] = (str(path), 8 + len(header) + offset, w)
    (directory / "config.json").write_text("{}")
    return written
