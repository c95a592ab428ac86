"""Host core: hash, router, serializer, checkpoint files.

Models: kraken/test/common/utils_test.cc, serialize_deserialize_test.cc of the
reference (round trips of every encodable type); the golden bytes below are
written out by hand from the wire rules.
"""
import os
import struct

import numpy as np
import pytest
import torch

from kraken_b200._native import C
from kraken_b200.utils.hashing import mix64, owner_of

M = (1 << 64) - 1


def py_mix64(v):
    v = (v * 3935559000370003845 + 2691343689449507681) & M
    v ^= v >> 21
    v ^= (v << 37) & M
    v ^= v >> 4
    v = (v * 4768777513237032717) & M
    v ^= (v << 20) & M
    v ^= v >> 41
    v ^= (v << 5) & M
    return v


def test_mix64_matches_formula():
    for v in [0, 1, 2, 12345, M, 1 << 63, 0xDEADBEEF]:
        assert C.mix64(v) == py_mix64(v)
    assert C.mix64_pair(3, 9) == py_mix64(3) ^ py_mix64(9)
    arr = np.array([0, 1, 12345, M], dtype=np.uint64)
    assert [int(x) for x in mix64(arr)] == [py_mix64(int(x)) for x in arr]


def test_owner_of_vectorised_matches_scalar():
    ids = torch.tensor([0, 1, -1, 1 << 40, 987654321], dtype=torch.int64)
    got = owner_of(7, ids, 5).tolist()
    want = [C.owner_of(7, int(i) & M, 5) for i in ids.tolist()]
    assert got == want


def test_router_ring_properties():
    r = C.Router()
    assert r.empty() and r.hit(5) == M
    assert r.add(0, "a") and r.add(1, "b")
    assert not r.add(1, "c")  # ids must strictly increase
    assert r.version() == 2 and r.node_ids() == [0, 1]
    vn = r.vnodes()
    assert len(vn) == 6 and [v[0] for v in vn] == sorted(v[0] for v in vn)
    # lookup = first vnode with hash >= hv, wrapping to the first one
    assert r.hit(vn[0][0]) == vn[0][1]
    assert r.hit(vn[2][0] + 1) == vn[3][1]
    assert r.hit(vn[-1][0] + 1) == vn[0][1]
    # every hash value is owned by exactly the node whose range covers it
    for hv in [0, 1, vn[1][0], vn[4][0] - 1, M]:
        owner = r.hit(hv)
        assert any(s < hv <= e or (s == 0 and hv == 0 and e == 0) or (hv <= e and s == 0)
                   for s, e in r.node_hash_ranges(owner))
    assert r.remove(0) and r.node_ids() == [1] and r.version() == 3


def test_router_binary_round_trip():
    r = C.Router.for_ranks(4)
    b = r.to_bytes()
    assert struct.unpack_from("<QQ", b) == (4, 4)  # version, node count
    r2 = C.Router.from_bytes(b)
    assert r2 == r and str(r2) == str(r)


def test_tensor_golden_bytes():
    t = torch.tensor([[1.0, 2.0, 3.0]], dtype=torch.float32)
    want = bytes([0]) + struct.pack("<Qqq", 2, 1, 3) + bytes([11]) + struct.pack("<fff", 1, 2, 3)
    assert C.serialize_tensor(t) == want
    assert torch.equal(C.deserialize_tensor(want), t)
    i = torch.tensor([5, -1], dtype=torch.int64)
    assert C.serialize_tensor(i) == bytes([0]) + struct.pack("<Qq", 1, 2) + bytes([9]) + struct.pack("<qq", 5, -1)


def test_string_conf_value_golden_bytes():
    assert C.serialize_string("ab") == struct.pack("<Q", 2) + b"ab"
    assert C.serialize_conf({"b": "2", "a": "1"}) == (struct.pack("<Q", 2) + struct.pack("<Q", 1) + b"a" +
                                                      struct.pack("<Q", 1) + b"1" + struct.pack("<Q", 1) + b"b" +
                                                      struct.pack("<Q", 1) + b"2")
    v = {"val": torch.tensor([1.5]), "states": {2: torch.tensor([0.25])}, "states_i": {0: 7}}
    row = lambda x: bytes([0]) + struct.pack("<Qq", 1, 1) + bytes([11]) + struct.pack("<f", x)
    want = row(1.5) + struct.pack("<Q", 1) + struct.pack("<I", 2) + row(0.25) + struct.pack("<Q", 1) + \
        struct.pack("<Iq", 0, 7)
    assert C.serialize_value(v) == want
    back = C.deserialize_value(want)
    assert torch.equal(back["val"], v["val"]) and back["states_i"] == {0: 7}


def test_coo_tensor_round_trip_densifies():
    b = C.serialize_coo(torch.tensor([[1, 3]]), torch.tensor([2.0, -1.0]), [5])
    assert b[0] == 1
    assert torch.equal(C.deserialize_tensor(b), torch.tensor([0.0, 2.0, 0.0, -1.0, 0.0]))


def test_truncated_input_raises():
    b = C.serialize_tensor(torch.ones(4))
    with pytest.raises(Exception):
        C.deserialize_tensor(b[:-3])


def test_model_meta_round_trip():
    m = C.ModelMeta()
    m.name = "m"
    m.optim_type = C.OptimType.kAdam
    m.optim_conf = {"beta1": "0.9"}
    t = C.TableMeta()
    t.id, t.name, t.table_type, t.dimension = 3, "emb", C.TableType.kSparse, 16
    t.init_type, t.init_conf = C.InitializerType.kNormal, {"mean": "0.0"}
    m.tables = {3: t}
    m2 = C.ModelMeta.from_bytes(m.to_bytes())
    assert m2.name == "m" and m2.optim_type == C.OptimType.kAdam and m2.tables[3].dimension == 16
    assert m2.tables[3].init_conf == {"mean": "0.0"}


def test_timestamp_dirs_and_retention(tmp_path):
    ok, k1 = C.ckpt_parse_timestamp("2024-01-02-03-04-05")
    ok2, k2 = C.ckpt_parse_timestamp("2024-01-02-03-04-06")
    assert ok and ok2 and k2 > k1
    assert not C.ckpt_parse_timestamp("not-a-date")[0]
    shard = tmp_path / "shard_0"
    for name in ["2020-01-01-00-00-00", "2021-01-01-00-00-00", "2022-01-01-00-00-00"]:
        (shard / name).mkdir(parents=True)
    new = C.ckpt_prepare_save_dir(str(tmp_path), 0, 3)
    kept = sorted(os.listdir(shard))
    assert len(kept) == 3 and "2020-01-01-00-00-00" not in kept and os.path.basename(new) in kept
    assert C.ckpt_latest_shard_dirs(str(tmp_path)) == {0: new}


def test_sparse_file_layout_and_filter(tmp_path):
    d = str(tmp_path)
    ids = torch.tensor([9, 8, 16, 1], dtype=torch.int64)
    vals = torch.arange(8, dtype=torch.float32).view(4, 2)
    st = {2: vals + 100}
    C.ckpt_save_sparse(d, 5, "t", 2, C.InitializerType.kConstant, {"value": "0"}, ids, vals, st, {0: torch.arange(4)})
    raw = open(os.path.join(d, "t.sparse"), "rb").read()
    assert raw[0] == 1 and struct.unpack_from("<Q", raw, 1)[0] == 5
    got = C.ckpt_load_sparse(d, "t")
    # slot = id % 8, ascending ids inside a slot: 8, 16 (slot 0) then 1, 9 (slot 1)
    assert got["ids"].tolist() == [8, 16, 1, 9]
    assert torch.equal(got["vals"], vals[[1, 2, 3, 0]])
    assert torch.equal(got["states"][2], (vals + 100)[[1, 2, 3, 0]])
    assert got["states_i"][0].tolist() == [1, 2, 3, 0]
    # modulo filter keeps exactly the rows OwnerOf assigns to the rank
    kept = []
    for rank in range(3):
        part = C.ckpt_load_sparse(d, "t", 1, 0, 3, rank)
        assert all(C.owner_of(0, i, 3) == rank for i in part["ids"].tolist())
        kept += part["ids"].tolist()
    assert sorted(kept) == [1, 8, 9, 16]


def test_dense_file_round_trip(tmp_path):
    v = {"val": torch.randn(3, 4), "states": {1: torch.randn(3, 4)}, "states_i": {0: 12}}
    C.ckpt_save_dense(str(tmp_path), 2, "w", v)
    back = C.ckpt_load_dense(str(tmp_path), "w")
    assert back["id"] == 2 and torch.equal(back["val"], v["val"]) and torch.equal(back["states"][1], v["states"][1])
    assert back["states_i"] == {0: 12}
    assert C.ckpt_load_dense(str(tmp_path), "missing") is None


def test_streamed_sparse_writer_and_fast_reader_match_the_plain_ones(tmp_path):
    """The multi-threaded stream writer must produce the same bytes as the plain writer, and the fast
    reader the same columns as the plain reader; a file whose rows differ in layout (as the reference
    writes them: state entries appear with the first update) must be left to the plain reader."""
    import torch
    from kraken_b200._native import C

    g = torch.Generator().manual_seed(3)
    n, dim = 20_000, 6
    ids = torch.randint(-(1 << 62), 1 << 62, (n,), generator=g, dtype=torch.int64).unique()
    n = ids.numel()
    vals = torch.randn(n, dim, generator=g)
    states = {3: torch.randn(n, dim, generator=g), 4: torch.rand(n, dim, generator=g)}
    steps = torch.randint(0, 50, (n,), generator=g, dtype=torch.int64)
    a, b = tmp_path / "plain", tmp_path / "stream"
    a.mkdir()
    b.mkdir()
    C.ckpt_save_sparse(str(a), 7, "emb.table", dim, C.InitializerType.kNormal, {"mean": "0", "stddev": "1"}, ids, vals,
                       states, {0: steps})
    w = C.SparseStreamWriter(str(b), 7, "emb.table", dim, C.InitializerType.kNormal, {"mean": "0", "stddev": "1"},
                             [3, 4], [0], 4)
    u = ids.numpy().view("uint64")
    for slot in range(8):
        sel = torch.from_numpy(((u % 8) == slot).nonzero()[0])
        sel = sel[torch.from_numpy(u[sel.numpy()].argsort())]
        w.begin_slot(int(sel.numel()))
        for lo in range(0, int(sel.numel()), 3000):   # several appends per slot
            s = sel[lo:lo + 3000]
            w.append(ids[s].contiguous(), vals[s].contiguous(), [states[3][s].contiguous(), states[4][s].contiguous()],
                     [steps[s].contiguous()])
    w.close()
    assert (a / "emb.table.sparse").read_bytes() == (b / "emb.table.sparse").read_bytes()
    fast = C.ckpt_load_sparse_fast(str(b), "emb.table", 3)
    plain = C.ckpt_load_sparse(str(a), "emb.table")
    assert fast is not False and fast is not None
    assert torch.equal(fast["ids"], plain["ids"]) and torch.equal(fast["vals"], plain["vals"])
    assert torch.equal(fast["states"][3], plain["states"][3]) and torch.equal(fast["states"][4], plain["states"][4])
    assert torch.equal(fast["states_i"][0], plain["states_i"][0])
    assert C.ckpt_load_sparse_fast(str(tmp_path), "missing") is None
    # the chunked reader: any row range of the file order, into caller-owned buffers that are reused
    rd = C.SparseChunkReader(str(b), "emb.table", 3)
    assert rd.exists and rd.fast and rd.rows == n and rd.dim == dim and rd.id == 7 and rd.name == "emb.table"
    assert list(rd.state_types) == [3, 4] and list(rd.int_state_types) == [0] and rd.init_conf == {"mean": "0", "stddev": "1"}
    cap = 4099
    bi, bv = torch.empty(cap, dtype=torch.int64), torch.empty(cap, dim)
    bs, bt = [torch.empty(cap, dim), torch.empty(cap, dim)], [torch.empty(cap, dtype=torch.int64)]
    for lo in list(range(0, n, cap)) + [n - 1, 5]:
        m = min(cap, n - lo)
        assert rd.read_into(lo, m, bi, bv, bs, bt) is True
        assert torch.equal(bi[:m], plain["ids"][lo:lo + m]) and torch.equal(bv[:m], plain["vals"][lo:lo + m])
        assert torch.equal(bs[0][:m], plain["states"][3][lo:lo + m]) and torch.equal(bs[1][:m], plain["states"][4][lo:lo + m])
        assert torch.equal(bt[0][:m], plain["states_i"][0][lo:lo + m])
    with pytest.raises(Exception):
        rd.read_into(n - 3, 10, bi, bv, bs, bt)          # beyond the end of the file
    assert not C.SparseChunkReader(str(tmp_path), "missing").exists
    # a row without state entries in the middle of the file: not the fixed layout
    raw = bytearray((a / "emb.table.sparse").read_bytes())
    row = w.row_bytes()
    first_row = len(raw) - int(w.bytes_written()) + 0  # both files are equal in length: header is what is not rows
    head = len(raw) - (n * row + 8 * 8)
    # rewrite the LAST row as {id, val, 0 states, 0 int states} and pad: length changes, so the layout check must fail
    cut = raw[:len(raw) - row] + raw[len(raw) - row:len(raw) - row + 8 + 18 + dim * 4] + (0).to_bytes(8, "little") * 2
    c = tmp_path / "mixed"
    c.mkdir()
    (c / "emb.table.sparse").write_bytes(bytes(cut))
    assert C.ckpt_load_sparse_fast(str(c), "emb.table") is False
    mixed_rd = C.SparseChunkReader(str(c), "emb.table")
    assert mixed_rd.exists and not mixed_rd.fast        # the file length does not fit rows of one size
    mixed = C.ckpt_load_sparse(str(c), "emb.table")
    assert mixed["ids"].numel() == n and float(mixed["states"][3][-1].abs().sum()) == 0.0
    assert head > 0 and first_row >= 0


def test_snappy_codec_reads_and_writes_the_block_format():
    """RPC bodies travel as Snappy streams (kraken/common/compress.h:18-91).  Streams assembled by hand
    from the format description - every element kind - must decode; what the compressor writes must
    decode to the input and must be made of the same elements; damaged streams are kSnappyUncompress."""
    un, co = C.snappy_uncompress, C.snappy_compress
    assert un(b"\x00") == b"" and co(b"") == b"\x00"
    assert co(b"abc") == b"\x03\x08abc"                                  # varint 3, literal of 3
    assert un(b"\x0c" + b"\x0cabcd" + b"\x11\x04") == b"abcd" * 3         # copy, 11-bit offset: length 8, offset 4
    assert un(b"\x09" + b"\x0cabcd" + b"\x12\x04\x00") == b"abcdabcda"    # copy, 16-bit offset: length 5
    assert un(b"\x09" + b"\x0cabcd" + b"\x13\x04\x00\x00\x00") == b"abcdabcda"   # copy, 32-bit offset
    assert un(b"\x0a" + b"\x00x" + b"\x15\x01") == b"x" * 10              # offset 1 < length 9: a run
    long_lit = bytes(range(256)) * 2                                      # 512 bytes: literal with 2 length bytes
    assert un(b"\x80\x04" + b"\xf4\xff\x01" + long_lit) == long_lit
    rng = np.random.default_rng(3)
    cases = [b"a" * 100_000, rng.integers(0, 256, 200_001, dtype=np.uint8).tobytes(),
             np.repeat(rng.normal(size=3000).astype(np.float32), 7).tobytes(),
             (b"0123456789abcdef" * 5000) + b"tail", bytes(70_000), b"ab" * 33, b"xyzw" * 17]
    for raw in cases:
        packed = co(raw)
        assert un(packed) == raw
    assert len(co(bytes(1 << 20))) < (1 << 20) // 20
    assert len(co(cases[1])) <= len(cases[1]) + len(cases[1]) // 6 + 32   # incompressible input stays within the bound
    for bad in (b"", b"\x05\x08abc", b"\x03\x08ab", b"\x04\x00a\x09\x02", b"\x04\x00a\x12\x00\x00", b"\x03\x08abcd",
                b"\xff\xff\xff\xff\xff\xff\x01"):
        with pytest.raises(C.KrakenError):
            un(bad)


def test_snappy_codec_interoperates_with_the_snappy_library():
    """Both directions against the Snappy build inside pyarrow (skipped where that is absent): the library
    reads what the codec writes and the codec reads what the library writes."""
    pa = pytest.importorskip("pyarrow")
    if not pa.Codec.is_available("snappy"):
        pytest.skip("pyarrow was built without snappy")
    lib = pa.Codec("snappy")
    rng = np.random.default_rng(11)
    for raw in (b"a" * 100_000, np.repeat(rng.normal(size=30_000).astype(np.float32), 3).tobytes(),
                rng.integers(0, 256, 70_001, dtype=np.uint8).tobytes(), b"0123456789abcdef" * 5000 + b"tail", b"", b"q"):
        assert C.snappy_uncompress(lib.compress(raw, asbytes=True)) == raw
        assert lib.decompress(C.snappy_compress(raw), decompressed_size=len(raw), asbytes=True) == raw
