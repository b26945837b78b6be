"""GGUF reader against a file written by the reference's own writer and read back by the reference's own reader (tests/golden/make_gguf.py): same tensor names,
dimensions, type names, bytes, data offset and key / value pairs; refusals for broken files (as tests/test_gguf_reader.py in the reference)."""
import json
import os
import struct

import numpy as np
import pytest

from kyojin_mac_b200 import foreign_gguf as GG

HERE = os.path.dirname(os.path.abspath(__file__))
PATH = os.path.join(HERE, "golden", "tiny.gguf")


@pytest.fixture(scope="module")
def gold():
    return np.load(os.path.join(HERE, "golden", "tiny_gguf.npz"))


def test_header_and_tensors_match_the_reference_reader(gold):
    with GG.GgufFile(PATH) as g:
        assert g.version == 3 and g.data_start == int(gold["data_start"])
        assert list(g.tensors) == [str(n) for n in gold["names"]]
        for i, (name, ti) in enumerate(g.tensors.items()):
            assert ti.ne == tuple(int(d) for d in gold[f"ne_{i}"]) and ti.tname == str(gold[f"type_{i}"])
            np.testing.assert_array_equal(np.asarray(g.raw(name)).reshape(-1), gold[f"raw_{i}"])
        want = json.loads(str(gold["kv_json"]))
        assert set(g.kv) == set(want)
        for k, v in want.items():
            got = g.kv[k]
            if isinstance(v, float):
                assert got == pytest.approx(v)
            elif isinstance(v, list) and v and isinstance(v[0], float):
                assert got == pytest.approx(v)
            else:
                assert got == v
        assert g.kv["general.alignment"] == 64 and g.data_start % 64 == 0
        assert g.raw("blk.0.ffn_gate_exps.weight").shape == (3, 16, 144) and g.tensors["blk.0.ffn_gate_exps.weight"].shape == (3, 16, 256)
        norm = g.array("blk.0.attn_norm.weight")
        assert norm.dtype == np.float32 and norm.shape == (64,)
        assert g.array("token_embd.weight").shape == (4, 32)
        with pytest.raises(GG.GgufTypeError):
            g.array("blk.0.attn_q.weight")                                  # a block format is not an array
        with pytest.raises(GG.GgufTypeError):
            g.load_pack("token_embd.weight")                                # no kernel format
        with pytest.raises(GG.GgufError):
            g.load_pack("blk.0.ffn_gate_exps.weight")                       # a stack, not a matrix


def test_packs_hold_the_stored_rows(gold):
    from oracle import kq_numpy as O
    with GG.GgufFile(PATH) as g:
        p = g.load_pack("blk.0.attn_q.weight")
        assert (p.fmt, p.n, p.k) == ("q4_k", 32, 512)
        np.testing.assert_array_equal(np.asarray(p.qs).reshape(-1), gold["raw_0"])
        ex = g.load_expert_packs("blk.0.ffn_gate_exps.weight")
        assert len(ex) == 3 and all((e.n, e.k) == (16, 256) for e in ex)
        raw = gold["raw_6"].reshape(3, 16, 144)
        for e in range(3):
            np.testing.assert_array_equal(np.asarray(ex[e].qs), raw[e])
        w = O.dequant("Q6_K", np.asarray(g.raw("blk.0.ffn_down.weight")), 256)   # the oracle decodes what the reader returns
        assert w.shape == (16, 256) and np.isfinite(w).all()


def test_split_shard_set_reads_as_one_file(gold, tmp_path):
    import shutil
    first = os.path.join(HERE, "golden", "tinysplit-00001-of-00002.gguf")
    with GG.GgufFile(first) as g:
        assert list(g.tensors) == [str(n) for n in gold["names"]]
        for i, name in enumerate(g.tensors):
            np.testing.assert_array_equal(np.asarray(g.raw(name)).reshape(-1), gold[f"raw_{i}"])       # bytes come from the shard that holds the tensor
        assert g.kv["general.architecture"] == "tiny" and g.kv["split.count"] == 2
    with pytest.raises(GG.GgufError):                                      # the second shard is not an entry point
        GG.GgufFile(os.path.join(HERE, "golden", "tinysplit-00002-of-00002.gguf"))
    lone = tmp_path / "tinysplit-00001-of-00002.gguf"
    shutil.copy(first, lone)
    with pytest.raises(GG.GgufError):                                      # a missing shard is an error, never a partial load
        GG.GgufFile(lone)
    renamed = tmp_path / "other.gguf"
    shutil.copy(first, renamed)
    with pytest.raises(GG.GgufError):
        GG.GgufFile(renamed)


def test_refusals(tmp_path):
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"NOPE" + b"\0" * 40)
    with pytest.raises(GG.GgufError):
        GG.GgufFile(bad)
    data = open(PATH, "rb").read()
    short = tmp_path / "short.gguf"
    short.write_bytes(data[:-100])                                          # the last tensor runs past the end
    with pytest.raises(GG.GgufError):
        GG.GgufFile(short)
    v9 = tmp_path / "v9.gguf"
    v9.write_bytes(data[:4] + struct.pack("<I", 9) + data[8:])
    with pytest.raises(GG.GgufError):
        GG.GgufFile(v9)
    hdr = tmp_path / "hdr.gguf"
    hdr.write_bytes(data[:40])                                              # header cut inside the key / value section
    with pytest.raises(GG.GgufError):
        GG.GgufFile(hdr)
