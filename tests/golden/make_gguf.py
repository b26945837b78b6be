"""Generates tests/golden/tiny.gguf with the REFERENCE's own writer (kyojin_mlx/foreign_synth.py:70-88 `write_gguf`) and tests/golden/tiny_gguf.npz with what the
reference's reader (kyojin_mlx/foreign_gguf.py:186-302 `GgufFile`) returns for it: names, shapes, type names, raw bytes and key / value pairs. Run in the build
container, where the reference is importable:  PYTHONPATH=<reference checkout> python tests/golden/make_gguf.py"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    from kyojin_mlx import foreign_gguf as GF, foreign_synth as FS
    rng = np.random.default_rng(2024)

    def blocks(tname, n, k):
        _, be, bb = next(v for v in GF.TYPES.values() if v[0] == tname)
        raw = rng.integers(0, 256, (n, k // be * bb), dtype=np.uint8)
        b = raw.reshape(n, k // be, bb)
        f16 = lambda: (np.abs(rng.standard_normal((n, k // be))) * 1e-2).astype("<f2").view(np.uint8).reshape(n, k // be, 2)
        if tname in ("Q4_K", "Q5_K"):
            b[..., 0:2], b[..., 2:4] = f16(), f16()
        elif tname == "Q8_0":
            b[..., 0:2] = f16()
        elif tname == "Q6_K":
            b[..., 208:210] = f16()
        elif tname == "Q3_K":
            b[..., 108:110] = f16()
        elif tname == "NVFP4":
            b[..., 0:4] = rng.integers(0x20, 0x48, (n, k // be, 4), dtype=np.uint8)
        return raw

    tensors = [
        ("blk.0.attn_q.weight", (512, 32), "Q4_K", blocks("Q4_K", 32, 512)),
        ("blk.0.ffn_down.weight", (256, 16), "Q6_K", blocks("Q6_K", 16, 256)),
        ("blk.0.attn_k.weight", (256, 16), "Q3_K", blocks("Q3_K", 16, 256)),
        ("blk.0.ffn_up.weight", (128, 16), "NVFP4", blocks("NVFP4", 16, 128)),
        ("blk.0.attn_norm.weight", (64,), "F32", rng.standard_normal(64).astype("<f4").view(np.uint8)),
        ("token_embd.weight", (32, 4), "F16", rng.standard_normal((4, 32)).astype("<f2").view(np.uint8)),
        ("blk.0.ffn_gate_exps.weight", (256, 16, 3), "Q4_K", blocks("Q4_K", 48, 256)),
        ("blk.0.attn_v.weight", (256, 16), "Q5_K", blocks("Q5_K", 16, 256)),
        ("blk.0.attn_output.weight", (256, 16), "Q8_0", blocks("Q8_0", 16, 256)),
    ]
    kv = {"general.architecture": "tiny", "general.name": "golden fixture", "tiny.block_count": 1, "tiny.rope.freq_base": 10000.0,
          "tokenizer.ggml.tokens": ["a", "b", "c"], "tiny.flag": True, "tiny.scores": [0.5, -1.0]}
    path = os.path.join(HERE, "tiny.gguf")
    FS.write_gguf(path, kv, tensors, align=64)
    g = GF.GgufFile(path)
    out = {"names": np.array(list(g.tensors)), "kv_json": np.array(json.dumps({k: (v if not isinstance(v, np.generic) else v.item()) for k, v in g.kv.items()}, default=lambda o: o.tolist() if hasattr(o, "tolist") else str(o)))}
    for i, (name, ti) in enumerate(g.tensors.items()):
        out[f"ne_{i}"] = np.array(ti.ne, np.int64)
        out[f"type_{i}"] = np.array(ti.tname)
        out[f"raw_{i}"] = np.array(g.raw(name)).reshape(-1)
    out["data_start"] = np.array(g.data_start)
    np.savez_compressed(os.path.join(HERE, "tiny_gguf.npz"), **out)
    print("wrote", path, os.path.getsize(path), "bytes;", len(g.tensors), "tensors; kv", list(g.kv))
    # a two-shard split set (gguf-split conventions: split.no / split.count / split.tensors.count, -0000i-of-0000N names)
    base = os.path.join(HERE, "tinysplit")
    FS.write_gguf(f"{base}-00001-of-00002.gguf", dict(kv, **{"split.no": 0, "split.count": 2, "split.tensors.count": len(tensors)}), tensors[:3])
    FS.write_gguf(f"{base}-00002-of-00002.gguf", {"split.no": 1, "split.count": 2, "split.tensors.count": len(tensors)}, tensors[3:])
    gs = GF.GgufFile(f"{base}-00001-of-00002.gguf")
    assert list(gs.tensors) == [t[0] for t in tensors]
    for i, name in enumerate(gs.tensors):
        assert np.array_equal(np.array(gs.raw(name)).reshape(-1), out[f"raw_{i}"]), name      # the reference reader sees the same bytes through the set
    print("wrote the split set", base, "-0000[12]-of-00002.gguf")


if __name__ == "__main__":
    sys.exit(main())
