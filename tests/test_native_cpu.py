"""Native host library: packer golden cases (restated from brain/src/feeder/packing.rs:119-188),
TKNS shards, row stream, safetensors, RNG streams."""
import ctypes as C
import os
import struct
import threading

import numpy as np
import pytest
import torch

from autoresearch_b200 import native

CAP = 2049


def _pack_all(docs, cap=CAP, buffer_docs=1000):
    lib = native.lib()
    p = lib.ar_packer_create(cap, buffer_docs)
    for d in docs:
        a = np.asarray(d, dtype=np.int32)
        lib.ar_packer_add_doc(p, a.ctypes.data, len(a))
    rows = []
    out = np.zeros(cap, dtype=np.uint16)
    while lib.ar_packer_next_row(p, 1, out.ctypes.data):
        rows.append(out.copy())
    lib.ar_packer_destroy(p)
    return rows


def test_packer_exact_fit():
    rows = _pack_all([[1] * CAP])
    assert len(rows) == 1 and (rows[0] == 1).all()


def test_packer_padding_on_exhaustion():
    rows = _pack_all([[42] * 100])
    assert len(rows) == 1 and (rows[0][:100] == 42).all() and (rows[0][100:] == 0).all()


def test_packer_crop_when_nothing_fits():
    rows = _pack_all([[1] * (CAP + 500), [2] * (CAP + 100)])
    assert len(rows) == 2 and (rows[0] == 2).all() and (rows[1] == 1).all()


def test_packer_best_fit_picks_largest_fitting():
    rows = _pack_all([[1] * 100, [2] * 1000, [3] * 2000])
    assert (rows[0][:2000] == 3).all() and (rows[0][2000:2049] == 1).all()


def test_packer_empty_source_and_multi_doc():
    assert _pack_all([]) == []
    rows = _pack_all([[1] * 1000, [2] * 1049])
    assert len(rows) == 1 and (rows[0][:1049] == 2).all() and (rows[0][1049:] == 1).all()


def test_packer_waits_for_refill_until_exhausted():
    lib = native.lib()
    p = lib.ar_packer_create(16, 4)
    a = np.arange(1, 6, dtype=np.int32)
    lib.ar_packer_add_doc(p, a.ctypes.data, 5)
    out = np.zeros(16, dtype=np.uint16)
    assert lib.ar_packer_next_row(p, 0, out.ctypes.data) == 0     # fewer than buffer_docs: wants more
    assert lib.ar_packer_next_row(p, 1, out.ctypes.data) == 1
    assert (out[:5] == a).all() and (out[5:] == 0).all()
    lib.ar_packer_destroy(p)


def test_shard_roundtrip_and_errors(tmp_path):
    from autoresearch_b200.data.shards import Shard, ShardLoader, write_shard
    rows = (np.arange(7 * 33).reshape(7, 33) % 500).astype(np.uint16)
    for i in range(3):
        write_shard(tmp_path / f"shard_{i:05d}.bin", rows + i, vocab=512)
    s = Shard(tmp_path / "shard_00001.bin")
    assert (s.vocab, s.seq_len, s.num_rows) == (512, 33, 7)
    assert (s.row(3) == rows[3] + 1).all()
    with pytest.raises(IndexError):
        s.row(7)
    bad = tmp_path / "shard_bad.bin"
    bad.write_bytes(b"NOPE" + struct.pack("<IIII", 1, 512, 33, 7))
    with pytest.raises(ValueError, match="magic"):
        Shard(bad)
    trunc = tmp_path / "shard_trunc.bin"
    trunc.write_bytes(b"TKNS" + struct.pack("<IIII", 1, 512, 33, 7) + b"\0" * 10)
    with pytest.raises(ValueError, match="truncated"):
        Shard(trunc)
    bad.unlink(); trunc.unlink()
    ld = ShardLoader(tmp_path, batch_size=2, seq_len=32, split="train")
    ids, tgt = ld.next_batch()
    assert ids.shape == (2, 32) and (ids[:, 1:] == tgt[:, :-1]).all()
    val = ShardLoader(tmp_path, batch_size=2, seq_len=32, split="val")
    assert len(val.files) == 1 and val.files[0].name == "shard_00002.bin"
    # rows shorter than SEQ+1 are concatenated
    ld2 = ShardLoader(tmp_path, batch_size=1, seq_len=50, split="val")
    ids2, _ = ld2.next_batch()
    assert ids2.shape == (1, 50) and ids2[0, 33].item() == int(rows[1, 0] + 2)


def test_shuffle_is_a_permutation_and_deterministic():
    from autoresearch_b200.data.shards import shuffle_order
    a, b = shuffle_order(17, 42), shuffle_order(17, 42)
    assert a == b and sorted(a) == list(range(17)) and a != list(range(17))
    assert shuffle_order(17, 43) != a


def test_row_stream_reads_rows_and_detects_truncation():
    from autoresearch_b200.data.shards import StdinRowStream
    T = 8
    r, w = os.pipe()
    rows = np.arange(6 * (T + 1), dtype=np.uint16).reshape(6, T + 1)

    def feed():
        os.write(w, rows.tobytes())
        os.close(w)

    th = threading.Thread(target=feed); th.start()
    s = StdinRowStream(batch_size=2, seq_len=T, fd=r, depth=2)
    got = []
    while True:
        b = s.next_batch(timeout_ms=5000)
        if b is None:
            break
        got.append((b[0].clone(), b[1].clone()))
    th.join()
    assert len(got) == 3 and s.rows_read() == 6
    assert (got[1][0].numpy() == rows[2:4, :-1]).all() and (got[1][1].numpy() == rows[2:4, 1:]).all()
    s.close()
    # a stream that ends in the middle of a row is an error, not a clean end
    r, w = os.pipe()
    os.write(w, rows.tobytes()[: 2 * (T + 1) * 2 + 5]); os.close(w)
    s = StdinRowStream(batch_size=2, seq_len=T, fd=r, depth=2)
    assert s.next_batch(timeout_ms=5000) is not None
    with pytest.raises(RuntimeError):
        s.next_batch(timeout_ms=5000)
    s.close()


def test_row_stream_timeout_when_feeder_is_silent():
    from autoresearch_b200.data.shards import StdinRowStream
    r, w = os.pipe()
    s = StdinRowStream(batch_size=1, seq_len=4, fd=r, depth=1)
    with pytest.raises(TimeoutError):
        s.next_batch(timeout_ms=100)
    os.close(w)
    s.close()


def test_safetensors_roundtrip_matches_library_reader(tmp_path):
    from autoresearch_b200.ckpt.safetensors_io import load_file, save_file
    t = {"b.weight": torch.randn(4, 6).to(torch.bfloat16), "a": torch.arange(5, dtype=torch.float32),
         "z.y": torch.randn(3, 2, 2)}
    p = tmp_path / "x.safetensors"
    save_file(t, str(p))
    back = load_file(str(p))
    assert set(back) == set(t)
    for k in t:
        assert back[k].dtype == t[k].dtype and torch.equal(back[k], t[k])
    st = pytest.importorskip("safetensors.torch")
    lib_read = st.load_file(str(p))
    for k in t:
        assert torch.equal(lib_read[k], t[k])
    st.save_file({k: v.contiguous() for k, v in t.items()}, str(tmp_path / "y.safetensors"))
    ours = load_file(str(tmp_path / "y.safetensors"))
    for k in t:
        assert torch.equal(ours[k], t[k])
    raw = p.read_bytes()
    n = struct.unpack("<Q", raw[:8])[0]
    assert n % 8 == 0 and raw[8:8 + n].lstrip().startswith(b'{"a":')      # sorted names, padded header


def test_safetensors_rejects_corrupt_files(tmp_path):
    from autoresearch_b200.ckpt.safetensors_io import load_file
    p = tmp_path / "bad.safetensors"
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(ValueError):
        load_file(str(p))
    hdr = b'{"a":{"dtype":"F32","shape":[4],"data_offsets":[0,16]}}'
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(ValueError, match="outside"):
        load_file(str(p))


def test_init_rng_streams_are_reproducible():
    from autoresearch_b200.models.init import InitRng
    a, b = InitRng(42), InitRng(42)
    u1, u2 = a.uniform((1000,), 0.5, torch.float32), b.uniform((1000,), 0.5, torch.float32)
    assert torch.equal(u1, u2) and u1.abs().max() <= 0.5 and u1.std() > 0.2
    n1 = a.normal((4001,), 1.0, torch.float32)
    assert abs(n1.mean().item()) < 0.1 and abs(n1.std().item() - 1.0) < 0.1
    # the xorshift64 recurrence itself: first draw from seed 42
    s = 42
    s ^= (s << 13) & (2**64 - 1); s ^= s >> 7; s ^= (s << 17) & (2**64 - 1)
    first = InitRng(42).uniform((1,), 1.0, torch.float32).item()
    assert abs(first - (2.0 * (s / 2**64) - 1.0)) < 1e-6


def test_synthetic_streams():
    from autoresearch_b200.data.synthetic import LcgStream, ZipfStream
    l = LcgStream(2, 16, vocab=8192)
    ids, tgt = l.next_batch()
    assert ids.min() >= 1 and ids.max() <= 8191 and (ids[:, 1:] == tgt[:, :-1]).all()
    st = 0xdeadbeef12345678
    st = (st * 6364136223846793005 + 1442695040888963407) % 2**64
    assert ids[0, 0].item() == (st >> 33) % 8191 + 1
    z1 = ZipfStream(2, 64, vocab=512, seed=7, rank=0, world=2)
    z2 = ZipfStream(4, 64, vocab=512, seed=7, rank=0, world=1)
    a, _ = z1.next_batch(); b, _ = z2.next_batch()
    assert torch.equal(a, b[:2])          # a rank sees its slice of the same global batch
    counts = torch.bincount(b.reshape(-1), minlength=512)
    assert counts[0] > counts[10] >= 0 and b.max() < 512
