"""CPU checks of the end-to-end harness: the synthetic GGUF writer produces a file with the layout the reference's loader
expects (src/gguf.cpp, src/model_common.cpp), and -- where the reference's CPU build of the driver exists -- the
reference's own model code loads it and runs deterministically."""
import json
import os
import struct
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "oracle", "e2e"))
import make_gguf  # noqa: E402

CPU_EXE = os.path.join(ROOT, "oracle", "_ref", "e2e_cpu")
SMALL = dict(arch="qwen2", n_layer=1, n_embd=256, n_head=2, n_kv=1, hd=128, n_ff=512, vocab=320, theta=1e6, bias=True)


def read_str(b, off):
    n = struct.unpack_from("<Q", b, off)[0]
    return b[off + 8: off + 8 + n].decode(), off + 8 + n


def test_gguf_writer_layout(tmp_path):
    path = str(tmp_path / "m.gguf")
    make_gguf.write_model(path, SMALL, seed=3)
    b = open(path, "rb").read()
    assert b[:4] == b"GGUF"
    version, n_tensors, n_kv = struct.unpack_from("<IQQ", b, 4)
    assert version == 3 and n_kv == 10
    off = 24
    meta = {}
    for _ in range(n_kv):
        key, off = read_str(b, off)
        typ = struct.unpack_from("<I", b, off)[0]
        off += 4
        if typ == 8:
            meta[key], off = read_str(b, off)
        elif typ == 4:
            meta[key] = struct.unpack_from("<I", b, off)[0]
            off += 4
        else:
            assert typ == 6
            meta[key] = struct.unpack_from("<f", b, off)[0]
            off += 4
    assert meta["general.architecture"] == "qwen2" and meta["qwen2.block_count"] == 1
    assert meta["qwen2.attention.head_count"] == 2 and meta["qwen2.attention.head_count_kv"] == 1
    tensors = {}
    for _ in range(n_tensors):
        name, off = read_str(b, off)
        nd = struct.unpack_from("<I", b, off)[0]
        dims = struct.unpack_from("<%dQ" % nd, b, off + 4)
        typ, toff = struct.unpack_from("<IQ", b, off + 4 + 8 * nd)
        off += 4 + 8 * nd + 12
        tensors[name] = (dims, typ, toff)
    data0 = (off + 31) // 32 * 32
    assert set(["token_embd.weight", "output_norm.weight", "blk.0.attn_q.weight", "blk.0.attn_k.bias",
                "blk.0.ffn_down.weight"]) <= set(tensors)
    end = 0
    for name, (dims, typ, toff) in tensors.items():
        assert toff % 32 == 0, name
        n = int(np.prod(dims))
        nbytes = n * 4 if typ == 0 else n // 32 * 34
        assert typ in (0, 8) and (typ == 0 or dims[0] % 32 == 0)
        end = max(end, toff + nbytes)
    assert data0 + end <= len(b) <= data0 + end + 32
    # one Q8_0 block of the embedding: fp16 scale then 32 int8
    dims, typ, toff = tensors["token_embd.weight"]
    assert dims == (256, 320) and typ == 8
    blk = b[data0 + toff: data0 + toff + 34]
    d = np.frombuffer(blk[:2], np.float16)[0]
    q = np.frombuffer(blk[2:], np.int8)
    assert 0 < float(d) < 1e-2 and np.abs(q.astype(np.int32)).max() <= 127
    # a norm weight is fp32 near 1
    dims, typ, toff = tensors["output_norm.weight"]
    w = np.frombuffer(b[data0 + toff: data0 + toff + 4 * dims[0]], np.float32)
    assert typ == 0 and abs(float(w.mean()) - 1.0) < 0.05


@pytest.mark.skipif(not os.path.exists(CPU_EXE), reason="oracle/_ref/e2e_cpu not built (reference tree absent at build time)")
def test_reference_cpu_model_runs_the_synthetic_file(tmp_path):
    path = str(tmp_path / "m.gguf")
    make_gguf.write_model(path, SMALL, seed=3)

    def run(tag):
        tok = str(tmp_path / (tag + ".tok"))
        lg = str(tmp_path / (tag + ".lg"))
        p = subprocess.run([CPU_EXE, "--model", path, "--prompt", "6", "--gen", "3", "--ctx", "64", "--batch", "4", "--tokens-out",
                            tok, "--logits-out", lg], capture_output=True, text=True, timeout=120)
        assert p.returncode == 0, p.stderr[-500:]
        line = json.loads([x for x in p.stdout.splitlines() if x.startswith("{")][-1])
        return line, np.fromfile(tok, np.int32), np.fromfile(lg, np.float32).reshape(2, -1)

    a, ta, la = run("a")
    b, tb, lb = run("b")
    assert a["n_prompt"] == 6 and a["n_gen"] == 3 and len(ta) == 4 and la.shape == (2, 320)
    assert np.array_equal(ta, tb) and np.array_equal(la, lb)         # deterministic
    assert np.isfinite(la).all() and la.std() > 0 and (0 <= ta).all() and (ta < 320).all()


def _reflib():
    from oracle.oracle import RefLib
    if not RefLib.available():
        pytest.skip("oracle/_ref/libref_attn.so not built (reference tree absent at build time)")
    lib = RefLib()
    if not hasattr(lib.L, "ref_dequantize_row"):
        pytest.skip("oracle/_ref/libref_attn.so predates ref_dequantize_row")
    return lib


@pytest.mark.parametrize("kind", ["q4_k", "q6_k"])
def test_k_quant_blocks_read_back_by_the_reference(kind):
    """The writer's Q4_K / Q6_K blocks, dequantised by the reference's own dequantize_row (src/model_cpu.cpp:70-88,
    114-140), give exactly the values the writer's restatement of those formulas gives, and those values are the
    N(0, 0.02)-like weights the writer means to produce."""
    lib = _reflib()
    rng = np.random.default_rng(11)
    rows, cols = 24, 1024
    if kind == "q4_k":
        raw = make_gguf.q4_k_bytes(rng, rows, cols)
        mine, typ = make_gguf.dequant_q4_k(raw), make_gguf.T_Q4_K
        assert raw.shape == (rows * cols // 256, 144)
    else:
        raw = make_gguf.q6_k_bytes(rng, rows, cols)
        mine, typ = make_gguf.dequant_q6_k(raw), make_gguf.T_Q6_K
        assert raw.shape == (rows * cols // 256, 210)
    ref = lib.dequantize_row(typ, raw.reshape(-1), rows * cols)
    assert np.array_equal(ref, mine.reshape(-1))
    assert abs(float(ref.mean())) < 2e-3 and 0.015 < float(ref.std()) < 0.025
    assert float(np.abs(ref).max()) < 0.12


def test_q4_k_m_file_layout(tmp_path):
    """The Q4_K_M-style mix: Q6_K for the embedding and for attn_v / ffn_down of the 'more bits' layers, Q4_K elsewhere,
    block-sized byte counts, 32-byte aligned offsets."""
    cfg = dict(arch="llama", n_layer=8, n_embd=256, n_head=2, n_kv=1, hd=128, n_ff=512, vocab=512, theta=5e5, bias=False)
    path = str(tmp_path / "m.gguf")
    make_gguf.write_model(path, cfg, seed=5, quant="q4_k_m")
    b = open(path, "rb").read()
    version, n_tensors, n_kv = struct.unpack_from("<IQQ", b, 4)
    off = 24
    for _ in range(n_kv):
        _, off = read_str(b, off)
        typ = struct.unpack_from("<I", b, off)[0]
        off += 4
        if typ == 8:
            _, off = read_str(b, off)
        else:
            off += 4
    types = {}
    for _ in range(n_tensors):
        name, off = read_str(b, off)
        nd = struct.unpack_from("<I", b, off)[0]
        dims = struct.unpack_from("<%dQ" % nd, b, off + 4)
        typ, toff = struct.unpack_from("<IQ", b, off + 4 + 8 * nd)
        off += 4 + 8 * nd + 12
        types[name] = typ
        assert toff % 32 == 0
    assert types["token_embd.weight"] == 14
    six = [i for i in range(8) if types["blk.%d.attn_v.weight" % i] == 14]
    assert six == [i for i in range(8) if make_gguf.more_bits(i, 8)] and 0 < len(six) < 8
    assert all(types["blk.%d.ffn_down.weight" % i] == types["blk.%d.attn_v.weight" % i] for i in range(8))
    assert all(types["blk.%d.attn_q.weight" % i] == 12 and types["blk.%d.ffn_gate.weight" % i] == 12 for i in range(8))


@pytest.mark.skipif(not os.path.exists(CPU_EXE), reason="oracle/_ref/e2e_cpu not built (reference tree absent at build time)")
def test_reference_cpu_model_runs_the_k_quant_file(tmp_path):
    cfg = dict(arch="llama", n_layer=2, n_embd=256, n_head=2, n_kv=1, hd=128, n_ff=512, vocab=512, theta=5e5, bias=False)
    path = str(tmp_path / "m.gguf")
    make_gguf.write_model(path, cfg, seed=5, quant="q4_k_m")
    tok, lg = str(tmp_path / "t"), str(tmp_path / "l")
    p = subprocess.run([CPU_EXE, "--model", path, "--prompt", "6", "--gen", "3", "--ctx", "64", "--batch", "4", "--tokens-out", tok,
                        "--logits-out", lg], capture_output=True, text=True, timeout=120)
    assert p.returncode == 0, p.stderr[-500:]
    la = np.fromfile(lg, np.float32).reshape(2, -1)
    assert la.shape == (2, 512) and np.isfinite(la).all() and la.std() > 0
