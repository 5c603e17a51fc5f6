"""The GGUF reader against damaged files (no GPU): a file written by gguf-py is truncated at many lengths and has
bytes of its header, metadata and tensor table overwritten at seeded positions. Every variant must either be declined
or open with a tensor table whose entries lie inside the file; querying every entry must not read outside the mapping.
Run in a child process so that a crash of the reader fails the test instead of the test session."""
import os
import subprocess
import sys

import numpy as np
import pytest

gguf = pytest.importorskip("gguf")

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import os, sys
import numpy as np
sys.path.insert(0, sys.argv[1])
from fucina_b200 import provider as P
path, out = sys.argv[2], sys.argv[3]
base = open(path, "rb").read()
size = len(base)
rng = np.random.default_rng(int(sys.argv[4]))
opened = declined = 0
def probe(data):
    global opened, declined
    with open(out, "wb") as f:
        f.write(data)
    try:
        g = P.Gguf(out)
    except P.Declined:
        declined += 1
        return
    opened += 1
    n = len(data)
    for i, t in enumerate(g.tensors()):
        assert t["offset"] + t["bytes"] <= n, (t, n)
        if t["bytes"]:
            g.data(i, min(t["bytes"], 64))                      # first bytes
            g.data(i, t["bytes"])[-1]                           # and the last one
        g.find(t["name"])
    for key in ("general.alignment", "general.name", "fucina.ptqtp.version", "tokenizer.ggml.tokens"):
        for fn in (g.meta_u64, g.meta_str):
            try:
                fn(key)
            except P.Declined:
                pass
    g.close()
# truncations: every length in the header / metadata / tensor table, then a few inside the data section
meta_end = int(sys.argv[5])
for cut in list(range(0, min(meta_end + 64, size), 7)) + [size - 1, size - 33, size // 2]:
    probe(base[:max(cut, 0)])
# overwritten bytes in the first part of the file (counts, lengths, types, offsets live there)
for _ in range(400):
    data = bytearray(base)
    for _ in range(int(rng.integers(1, 4))):
        pos = int(rng.integers(0, meta_end))
        width = int(rng.choice([1, 4, 8]))
        val = rng.choice([0, 1, 0xff, 0x7f, 0x80, int(rng.integers(0, 256))])
        for j in range(width):
            if pos + j < size:
                data[pos + j] = int(val) if j == 0 or val in (0, 0xff) else int(rng.integers(0, 256))
    probe(bytes(data))
print("opened", opened, "declined", declined)
"""


def test_damaged_files_are_declined_or_read_inside_bounds(tmp_path):
    from parity import make_weights

    QT = gguf.GGMLQuantizationType
    path = str(tmp_path / "small.gguf")
    w = gguf.GGUFWriter(path, "llama")
    w.add_string("general.name", "fuzz")
    w.add_uint32("fucina.ptqtp.version", 1)
    w.add_array("tokenizer.ggml.tokens", ["a", "bc", "def"])
    w.add_tensor("blk.0.attn_q.weight", make_weights("q4_k", 8, 256, 1), raw_dtype=QT.Q4_K)
    w.add_tensor("blk.0.attn_k.weight", make_weights("q8_0", 4, 64, 2), raw_dtype=QT.Q8_0)
    w.add_tensor("token_embd.weight", np.arange(32, dtype=np.float32).reshape(4, 8))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    reader = gguf.GGUFReader(path)
    meta_end = int(min(t.data_offset for t in reader.tensors))
    del reader
    r = subprocess.run([sys.executable, "-c", CHILD, ROOT, path, str(tmp_path / "variant.gguf"), "1234", str(meta_end)],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, f"reader crashed or broke a bound (exit {r.returncode}):\n{r.stdout[-2000:]}\n{r.stderr[-4000:]}"
    opened, declined = (int(x) for x in r.stdout.split()[1::2])
    assert declined > 50 and opened + declined > 400   # most damage is caught; some leaves a readable file
