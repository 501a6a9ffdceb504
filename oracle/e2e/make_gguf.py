"""Writes a synthetic GGUF model file that the reference's loader accepts (src/gguf.cpp, src/model_common.cpp).

TEST INFRASTRUCTURE.  There are no real checkpoints here; the end-to-end drop-in check runs the reference's own model
code on random-init weights of a named architecture:
    qwen2-1.5b   28 layers, n_embd 1536, 12/2 heads of 128, n_ff 8960, vocab 151936, rope theta 1e6 (neox), q/k/v biases
    llama3-8b    32 layers, n_embd 4096, 32/8 heads of 128, n_ff 14336, vocab 128256, rope theta 5e5 (normal)
    tiny         2 layers of the qwen2 shape with a 4096-token vocabulary (what the CPU build can run in seconds)
All matrices are Q8_0 (34-byte blocks: fp16 scale, 32 int8) with values ~ N(0, 0.02); norm weights are
1 + N(0, 0.05) in fp32; biases N(0, 0.1).  Seeded, so every build of the reference reads the same file.

    python oracle/e2e/make_gguf.py --arch tiny --out /tmp/tiny.gguf [--layers N] [--seed S]
"""
import argparse
import struct

import numpy as np

ARCHS = {
    "qwen2-1.5b": dict(arch="qwen2", n_layer=28, n_embd=1536, n_head=12, n_kv=2, hd=128, n_ff=8960, vocab=151936,
                       theta=1e6, bias=True),
    "llama3-8b": dict(arch="llama", n_layer=32, n_embd=4096, n_head=32, n_kv=8, hd=128, n_ff=14336, vocab=128256,
                      theta=5e5, bias=False),
    "tiny": dict(arch="qwen2", n_layer=2, n_embd=1536, n_head=12, n_kv=2, hd=128, n_ff=8960, vocab=4096, theta=1e6,
                 bias=True),
}
T_F32, T_Q8_0 = 0, 8                       # ggml type numbers (src/common.h: enum DType)
GT_U32, GT_F32, GT_STR = 4, 6, 8           # GGUF metadata value types
ALIGN = 32


def gstr(s):
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def kv_u32(k, v):
    return gstr(k) + struct.pack("<II", GT_U32, v)


def kv_f32(k, v):
    return gstr(k) + struct.pack("<If", GT_F32, v)


def kv_str(k, v):
    return gstr(k) + struct.pack("<I", GT_STR) + gstr(v)


def q8_0_bytes(rng, rows, cols, std=0.02):
    """rows x cols matrix as Q8_0 blocks.  int8 ~ round(N(0,1) * 40) clipped, fp16 scale std/40 per block."""
    assert cols % 32 == 0
    nblk = rows * cols // 32
    out = np.empty((nblk, 34), np.uint8)
    d = np.float16(std / 40.0)
    out[:, 0:2] = np.frombuffer(d.tobytes(), np.uint8)
    step = 1 << 20
    for b0 in range(0, nblk, step):
        n = min(step, nblk - b0)
        q = np.clip(np.rint(rng.standard_normal((n, 32), dtype=np.float32) * 40.0), -127, 127).astype(np.int8)
        out[b0:b0 + n, 2:] = q.view(np.uint8)
    return out


def write_model(path, cfg, seed=1234, n_ctx=8192):
    rng = np.random.default_rng(seed)
    a = cfg["arch"]
    ne, nh, nkv, hd, nff, vocab = cfg["n_embd"], cfg["n_head"], cfg["n_kv"], cfg["hd"], cfg["n_ff"], cfg["vocab"]
    meta = [
        kv_str("general.architecture", a), kv_u32("general.alignment", ALIGN),
        kv_u32(a + ".block_count", cfg["n_layer"]), kv_u32(a + ".attention.head_count", nh),
        kv_u32(a + ".attention.head_count_kv", nkv), kv_u32(a + ".attention.key_length", hd),
        kv_u32(a + ".rope.dimension_count", hd), kv_f32(a + ".rope.freq_base", cfg["theta"]),
        kv_f32(a + ".attention.layer_norm_rms_epsilon", 1e-6), kv_u32(a + ".context_length", n_ctx),
    ]
    tensors = []        # (name, dims (ne0 first), type, generator)

    def mat(name, n_in, n_out):
        tensors.append((name, (n_in, n_out), T_Q8_0, lambda: q8_0_bytes(rng, n_out, n_in)))

    def vec(name, n, kind):
        if kind == "norm":
            tensors.append((name, (n,), T_F32, lambda: (1.0 + 0.05 * rng.standard_normal(n)).astype(np.float32)))
        else:
            tensors.append((name, (n,), T_F32, lambda: (0.1 * rng.standard_normal(n)).astype(np.float32)))

    mat("token_embd.weight", ne, vocab)
    vec("output_norm.weight", ne, "norm")
    for i in range(cfg["n_layer"]):
        p = "blk.%d." % i
        vec(p + "attn_norm.weight", ne, "norm")
        mat(p + "attn_q.weight", ne, nh * hd)
        mat(p + "attn_k.weight", ne, nkv * hd)
        mat(p + "attn_v.weight", ne, nkv * hd)
        mat(p + "attn_output.weight", nh * hd, ne)
        vec(p + "ffn_norm.weight", ne, "norm")
        mat(p + "ffn_gate.weight", ne, nff)
        mat(p + "ffn_up.weight", ne, nff)
        mat(p + "ffn_down.weight", nff, ne)
        if cfg["bias"]:
            vec(p + "attn_q.bias", nh * hd, "bias")
            vec(p + "attn_k.bias", nkv * hd, "bias")
            vec(p + "attn_v.bias", nkv * hd, "bias")

    def nbytes(dims, typ):
        n = int(np.prod(dims))
        return n * 4 if typ == T_F32 else n // 32 * 34

    infos, off = [], 0
    for name, dims, typ, _ in tensors:
        infos.append(gstr(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) +
                     struct.pack("<IQ", typ, off))
        off = (off + nbytes(dims, typ) + ALIGN - 1) // ALIGN * ALIGN
    head = b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(meta)) + b"".join(meta) + b"".join(infos)
    with open(path, "wb") as f:
        f.write(head)
        f.write(b"\0" * ((-len(head)) % ALIGN))
        for name, dims, typ, gen in tensors:
            data = gen().tobytes()
            assert len(data) == nbytes(dims, typ), name
            f.write(data)
            f.write(b"\0" * ((-len(data)) % ALIGN))
    return off


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--arch", default="tiny", choices=sorted(ARCHS))
    ap.add_argument("--out", required=True)
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--seed", type=int, default=1234)
    args = ap.parse_args()
    cfg = dict(ARCHS[args.arch])
    if args.layers:
        cfg["n_layer"] = args.layers
    n = write_model(args.out, cfg, args.seed)
    print("wrote %s: %s, %d layers, %.1f MB of tensor data" % (args.out, args.arch, cfg["n_layer"], n / 1e6))


if __name__ == "__main__":
    main()
