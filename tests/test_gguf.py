"""GGUF file -> resident weights (the reference: src/gguf.zig parsing, src/weights.zig:2621-2816 residency,
src/ptqtp_gguf.zig plane naming). Files are written here with gguf-py, so the reader is checked against an independent
writer; opening and querying need no GPU, loading does."""
import os

import numpy as np
import pytest

import oracle
from parity import make_weights

gguf = pytest.importorskip("gguf")
QT = gguf.GGMLQuantizationType


def _write(path, tensors, meta=(), alignment=None):
    w = gguf.GGUFWriter(path, "llama")
    if alignment:
        w.add_custom_alignment(alignment)
    for key, val in meta:
        if isinstance(val, str):
            w.add_string(key, val)
        elif isinstance(val, list):
            w.add_array(key, val)
        else:
            w.add_uint32(key, val)
    for name, arr, qt in tensors:
        w.add_tensor(name, arr, raw_dtype=qt)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    """A small file with every served format, a plain tensor, an expert stack and PTQTP planes."""
    rng = np.random.default_rng(41)
    t = {
        "blk.0.attn_q.weight": (make_weights("q4_k", 96, 512, 1), QT.Q4_K, (96, 512)),
        "blk.0.attn_k.weight": (make_weights("q8_0", 64, 256, 2), QT.Q8_0, (64, 256)),
        "blk.0.attn_v.weight": (make_weights("q6_k", 40, 256, 3), QT.Q6_K, (40, 256)),
        "output.weight": (make_weights("q4_k", 200, 2048, 4), QT.Q4_K, (200, 2048)),   # tile-major on the device
        "blk.0.ffn_gate_exps.weight": (make_weights("q5_k", 4 * 32, 256, 5).reshape(4, 32, -1), QT.Q5_K, (4, 32, 256)),
        "blk.0.ffn_down.weight.ptqtp0": (make_weights("tq2_0", 68, 512, 6), QT.TQ2_0, (68, 512)),
        "blk.0.ffn_down.weight.ptqtp1": (make_weights("tq2_0", 68, 512, 7), QT.TQ2_0, (68, 512)),
        "blk.1.bad.ptqtp0": (make_weights("tq2_0", 8, 256, 8), QT.TQ2_0, (8, 256)),
        "blk.1.bad.ptqtp2": (make_weights("tq2_0", 8, 256, 9), QT.TQ2_0, (8, 256)),
        "token_embd.weight": (rng.standard_normal((16, 64)).astype(np.float32), None, (16, 64)),
    }
    path = str(tmp_path_factory.mktemp("gguf") / "model.gguf")
    _write(path, [(n, a, q) for n, (a, q, _) in t.items()],
           meta=[("fucina.ptqtp.version", 1), ("general.name", "parity model"), ("tokenizer.ggml.tokens", ["a", "bc", "def"])])
    return path, t


def test_tensor_table_and_metadata_match_the_writer(model):
    from fucina_b200 import provider as P

    path, t = model
    g = P.Gguf(path)
    listed = {x["name"]: x for x in g.tensors()}
    assert set(listed) == set(t)
    reader = gguf.GGUFReader(path)
    theirs = {x.name: x for x in reader.tensors}
    for name, (arr, qt, shape) in t.items():
        mine = listed[name]
        assert mine["ggml_type"] == int(theirs[name].tensor_type)
        assert mine["offset"] == int(theirs[name].data_offset)
        assert mine["bytes"] == arr.nbytes
        assert mine["dims"] == list(shape)[::-1]                     # GGUF stores the innermost dimension first
        assert mine["fmt"] == (-1 if qt is None else {QT.Q4_K: 2, QT.Q8_0: 0, QT.Q6_K: 1, QT.Q5_K: 3, QT.TQ2_0: 16}[qt])
        assert np.array_equal(g.data(g.find(name), arr.nbytes), np.ascontiguousarray(arr).view(np.uint8).reshape(-1))
    assert g.find("no.such.tensor") == -1
    assert g.meta_u64("fucina.ptqtp.version") == 1
    assert g.meta_str("general.name") == "parity model"
    with pytest.raises(P.Declined):
        g.meta_u64("general.alignment")     # absent: the default of 32 applies (offsets above agree with the writer's)
    with pytest.raises(P.Declined):
        g.meta_u64("general.name")
    g.close()


def test_custom_alignment_and_malformed_files(tmp_path):
    from fucina_b200 import provider as P

    path = str(tmp_path / "a64.gguf")
    blocks = make_weights("q8_0", 4, 64, 11)
    _write(path, [("w", blocks, QT.Q8_0), ("v", blocks, QT.Q8_0)], alignment=64)
    g = P.Gguf(path)
    ts = g.tensors()
    assert all(x["offset"] % 64 == 0 for x in ts) and ts[1]["offset"] - ts[0]["offset"] == 320  # 272 bytes padded to 64
    assert np.array_equal(g.data(1, blocks.size), blocks.reshape(-1))
    g.close()
    raw = open(path, "rb").read()
    bad = str(tmp_path / "bad.gguf")
    for content in (b"GGUX" + raw[4:], raw[:40], raw[: len(raw) - 100], raw[:4] + (9).to_bytes(4, "little") + raw[8:]):
        open(bad, "wb").write(content)
        with pytest.raises(P.Declined):
            P.Gguf(bad)
    with pytest.raises(P.Declined):
        P.Gguf(str(tmp_path / "missing.gguf"))


def test_row_shards_cover_the_rows():
    from fucina_b200 import provider as P

    for n, ranks in ((32000, 8), (11008, 8), (200, 4), (31, 2), (4096, 3)):
        spans = [P.shard_rows(n, ranks, r) for r in range(ranks)]
        assert spans[0][0] == 0 and sum(rows for _, rows in spans) == n
        for (a0, ar), (b0, _) in zip(spans, spans[1:]):
            assert a0 + ar == b0 and (ar == 0 or a0 % 32 == 0)


@pytest.mark.gpu
def test_resident_weights_hold_the_file_bytes(model):
    from fucina_b200 import provider as P

    P.init(0)
    path, t = model
    g = P.Gguf(path)
    for name, (arr, qt, shape) in t.items():
        if qt is None or "bad" in name:
            continue
        w = g.load_weights(name)
        assert np.array_equal(w.download_gguf().reshape(-1), np.ascontiguousarray(arr).view(np.uint8).reshape(-1)), name
        w.free()
    # the shard of a column-sharded linear (tile-major: 32-row boundaries) and of an expert stack
    out = t["output.weight"][0]
    r0, rows = P.shard_rows(200, 4, 1)
    w = g.load_weights("output.weight", r0, rows)
    assert (r0, rows) == (64, 64) and np.array_equal(w.download_gguf(), out[64:128])
    w.free()
    stack = t["blk.0.ffn_gate_exps.weight"][0]
    w = g.load_weights("blk.0.ffn_gate_exps.weight", 0, 0, 2, 2)
    assert w.n_mats == 2 and np.array_equal(w.download_gguf().reshape(2, 32, -1), stack[2:4])
    w.free()
    w = g.load_weights("blk.0.ffn_gate_exps.weight", 8, 16, 1, 3)     # rows 8..23 of experts 1..3
    assert np.array_equal(w.download_gguf().reshape(3, 16, -1), stack[1:4, 8:24])
    w.free()
    with pytest.raises(P.Declined):
        g.load_weights("token_embd.weight")                          # not a quantized format
    with pytest.raises(P.Declined):
        g.load_weights("output.weight", 190, 20)                     # rows past the end
    g.close()


@pytest.mark.gpu
def test_a_tensor_larger_than_the_staging_buffers(tmp_path):
    # several 32 MiB chunks, the last one ragged, through both staging buffers
    from fucina_b200 import provider as P

    P.init(0)
    n, k = 33000, 4096
    rng = np.random.default_rng(43)
    blocks = rng.integers(0, 256, size=(n, k // 256 * 144), dtype=np.uint8)
    path = str(tmp_path / "big.gguf")
    _write(path, [("lm_head", blocks, QT.Q4_K)])
    g = P.Gguf(path)
    w = g.load_weights("lm_head")
    assert np.array_equal(w.download_gguf(), blocks)
    w.free()
    g.close()


@pytest.mark.gpu
def test_ptqtp_planes_load_in_order_and_multiply(model):
    import torch

    from fucina_b200 import provider as P
    from parity import TOL_INT8, assert_close

    P.init(0)
    path, t = model
    g = P.Gguf(path)
    planes = g.load_ptqtp_planes("blk.0.ffn_down.weight")
    assert len(planes) == 2
    ps = [t["blk.0.ffn_down.weight.ptqtp0"][0], t["blk.0.ffn_down.weight.ptqtp1"][0]]
    for w, b in zip(planes, ps):
        assert np.array_equal(w.download_gguf(), b)
    a = np.random.default_rng(44).standard_normal((2, 512)).astype(np.float32)
    cd = torch.full((2, 68), float("nan"), dtype=torch.float32, device="cuda")
    P.gemm_ptqtp_dev(planes, torch.from_numpy(a).cuda(), cd, 2)
    P.synchronize()
    assert_close(cd.cpu().numpy(), oracle.matmul_ptqtp(ps, a), TOL_INT8, "ptqtp planes from a file")
    with pytest.raises(P.Declined):
        g.load_ptqtp_planes("blk.1.bad")            # plane 2 without plane 1 (src/ptqtp_gguf.zig:66)
    with pytest.raises(P.Declined):
        g.load_ptqtp_planes("blk.0.attn_q.weight")  # no planes under this name
    for w in planes:
        w.free()
    g.close()
