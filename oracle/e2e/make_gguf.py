"""Writes a synthetic GGUF model file that the reference's loader accepts (src/gguf.cpp, src/model_common.cpp).

TEST INFRASTRUCTURE.  There are no real checkpoints here; the end-to-end drop-in check runs the reference's own model
code on random-init weights of a named architecture:
    qwen2-1.5b   28 layers, n_embd 1536, 12/2 heads of 128, n_ff 8960, vocab 151936, rope theta 1e6 (neox), q/k/v biases
    llama3-8b    32 layers, n_embd 4096, 32/8 heads of 128, n_ff 14336, vocab 128256, rope theta 5e5 (normal)
    tiny         2 layers of the qwen2 shape with a 4096-token vocabulary (what the CPU build can run in seconds)
Matrices are Q8_0 (34-byte blocks: fp16 scale, 32 int8) by default, or -- with --quant q4_k_m -- the mix a Q4_K_M
file carries: Q4_K everywhere except Q6_K for the token embedding (which is also the output head) and for attn_v and
ffn_down of the first and last eighth of the layers and every third layer in between.  Values ~ N(0, 0.02) in every
format; norm weights are 1 + N(0, 0.05) in fp32; biases N(0, 0.1).  Seeded, so every build of the reference reads the
same file.  The K-quant blocks are written from the block layouts (src/quant.h:12-43) and read back by
dequant_q4_k / dequant_q6_k below, which restate the reference's dequantisation (src/model_cpu.cpp:38-46, 70-88,
114-140); tests/test_e2e_cpu.py checks them against the reference's own dequantize_row.

    python oracle/e2e/make_gguf.py --arch tiny --out /tmp/tiny.gguf [--layers N] [--seed S] [--quant q8_0|q4_k_m]
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
T_F32, T_Q8_0, T_Q4_K, T_Q6_K = 0, 8, 12, 14     # ggml type numbers (src/common.h: enum DType)
BLOCK = {T_Q8_0: (32, 34), T_Q4_K: (256, 144), T_Q6_K: (256, 210)}   # elements, bytes per block
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


_BITS16 = np.array([bin(i).count("1") for i in range(65536)], np.uint8)
_LUT_Q4 = _BITS16[np.arange(65536) & 0x7FFF]                      # Binomial(15, 1/2): 0..15, mean 7.5, sd 1.936
_a = np.arange(65536)
_LUT_Q6 = ((_a & 15) + ((_a >> 4) & 15) + ((_a >> 8) & 15) + (_a >> 12) + 2).astype(np.uint8)   # 2..62, mean 32, sd 9.22


def q4_k_bytes(rng, rows, cols, std=0.02):
    """rows x cols matrix as Q4_K blocks (144 bytes: fp16 d, fp16 dmin, 12 bytes of packed 6-bit scales and mins, 128
    bytes of nibbles; x = d*sc*q - dmin*m).  The fields are drawn directly: q ~ Binomial(15, 1/2) (bell-shaped over
    0..15; sixteen random bits per element through a table, which is what makes an 8-billion-element file quick to
    write), per 32 elements a scale sc in 28..36 and the min m = sc, d and dmin fixed so that d*sc*7.5 = dmin*m (zero
    mean) and d*32*sd(q) = std."""
    assert cols % 256 == 0
    nblk = rows * cols // 256
    out = np.empty((nblk, 144), np.uint8)
    d = np.float16(std / (32.0 * 1.936))
    dmin = np.float16(float(d) * 7.5)
    out[:, 0:2] = np.frombuffer(d.tobytes(), np.uint8)
    out[:, 2:4] = np.frombuffer(dmin.tobytes(), np.uint8)
    step = 1 << 16
    for b0 in range(0, nblk, step):
        n = min(step, nblk - b0)
        sc = rng.integers(28, 37, size=(n, 8), dtype=np.uint8)
        m = sc
        sb = np.empty((n, 12), np.uint8)
        sb[:, 0:4] = (sc[:, 0:4] & 63) | ((sc[:, 4:8] >> 4) << 6)
        sb[:, 4:8] = (m[:, 0:4] & 63) | ((m[:, 4:8] >> 4) << 6)
        sb[:, 8:12] = (sc[:, 4:8] & 0xF) | ((m[:, 4:8] & 0xF) << 4)
        out[b0:b0 + n, 4:16] = sb
        q = _LUT_Q4[rng.integers(0, 65536, size=(n, 4, 2, 32), dtype=np.uint16)]
        # 64 elements share 32 bytes: the first 32 in the low nibbles, the next 32 in the high nibbles
        out[b0:b0 + n, 16:] = (q[:, :, 0, :] | (q[:, :, 1, :] << 4)).reshape(n, 128)
    return out


def dequant_q4_k(blocks):
    """[nblk][144] uint8 -> [nblk][256] fp32, the arithmetic of dequantize_row_q4_K (src/model_cpu.cpp:70-88)."""
    b = np.ascontiguousarray(blocks)
    d = b[:, 0:2].copy().view(np.float16).astype(np.float32)[:, 0]
    dmin = b[:, 2:4].copy().view(np.float16).astype(np.float32)[:, 0]
    sb = b[:, 4:16]
    sc = np.empty((b.shape[0], 8), np.uint8)
    m = np.empty_like(sc)
    sc[:, 0:4] = sb[:, 0:4] & 63
    m[:, 0:4] = sb[:, 4:8] & 63
    sc[:, 4:8] = (sb[:, 8:12] & 0xF) | ((sb[:, 0:4] >> 6) << 4)
    m[:, 4:8] = (sb[:, 8:12] >> 4) | ((sb[:, 4:8] >> 6) << 4)
    qs = b[:, 16:].reshape(-1, 4, 32)
    q = np.stack([qs & 0xF, qs >> 4], axis=2).reshape(-1, 8, 32).astype(np.float32)
    d1 = (d[:, None] * sc.astype(np.float32))[:, :, None]
    m1 = (dmin[:, None] * m.astype(np.float32))[:, :, None]
    return (d1 * q - m1).reshape(-1, 256).astype(np.float32)


def q6_k_bytes(rng, rows, cols, std=0.02):
    """rows x cols matrix as Q6_K blocks (210 bytes: 128 bytes of low nibbles, 64 bytes of high bit pairs, 16 int8
    scales, fp16 d; x = d*sc*q with q in -32..31).  Drawn directly: q + 32 = 2 + the sum of four random nibbles
    (bell-shaped over 2..62, sd 9.22), one scale in 28..36 per 16 elements, d fixed so that d*32*sd(q) = std."""
    assert cols % 256 == 0
    nblk = rows * cols // 256
    out = np.empty((nblk, 210), np.uint8)
    d = np.float16(std / (32.0 * 9.22))
    out[:, 208:210] = np.frombuffer(d.tobytes(), np.uint8)
    step = 1 << 16
    for b0 in range(0, nblk, step):
        n = min(step, nblk - b0)
        out[b0:b0 + n, 192:208] = rng.integers(28, 37, size=(n, 16), dtype=np.int8).view(np.uint8)
        # element (half h, group g of 32, lane l) -> 6-bit value v = q + 32
        v = _LUT_Q6[rng.integers(0, 65536, size=(n, 2, 4, 32), dtype=np.uint16)]
        lo, hi = v & 0xF, v >> 4
        ql = np.empty((n, 2, 2, 32), np.uint8)          # [half][which 32 bytes][l]: groups 0,2 share bytes, groups 1,3 too
        ql[:, :, 0, :] = lo[:, :, 0, :] | (lo[:, :, 2, :] << 4)
        ql[:, :, 1, :] = lo[:, :, 1, :] | (lo[:, :, 3, :] << 4)
        out[b0:b0 + n, 0:128] = ql.reshape(n, 128)
        qh = hi[:, :, 0, :] | (hi[:, :, 1, :] << 2) | (hi[:, :, 2, :] << 4) | (hi[:, :, 3, :] << 6)
        out[b0:b0 + n, 128:192] = qh.reshape(n, 64)
    return out


def dequant_q6_k(blocks):
    """[nblk][210] uint8 -> [nblk][256] fp32, the arithmetic of dequantize_row_q6_K (src/model_cpu.cpp:114-140)."""
    b = np.ascontiguousarray(blocks)
    n = b.shape[0]
    ql = b[:, 0:128].reshape(n, 2, 2, 32)
    qh = b[:, 128:192].reshape(n, 2, 32)
    sc = b[:, 192:208].copy().view(np.int8).reshape(n, 2, 8).astype(np.float32)
    d = b[:, 208:210].copy().view(np.float16).astype(np.float32)[:, 0]
    v = np.empty((n, 2, 4, 32), np.int32)
    v[:, :, 0, :] = (ql[:, :, 0, :] & 0xF) | (((qh >> 0) & 3) << 4)
    v[:, :, 1, :] = (ql[:, :, 1, :] & 0xF) | (((qh >> 2) & 3) << 4)
    v[:, :, 2, :] = (ql[:, :, 0, :] >> 4) | (((qh >> 4) & 3) << 4)
    v[:, :, 3, :] = (ql[:, :, 1, :] >> 4) | (((qh >> 6) & 3) << 4)
    q = (v - 32).astype(np.float32)
    # scale of (group g, lane l) is sc[2*g + l // 16]
    s = np.repeat(sc.reshape(n, 2, 4, 2), 16, axis=3)
    return ((d[:, None, None, None] * s) * q).reshape(n, 256).astype(np.float32)


def more_bits(i, n):
    """Layers whose attn_v and ffn_down are kept in Q6_K in the Q4_K_M mix."""
    return i < n // 8 or i >= 7 * n // 8 or (i - n // 8) % 3 == 2


def write_model(path, cfg, seed=1234, n_ctx=8192, quant="q8_0"):
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

    def mat(name, n_in, n_out, six=False):
        if quant == "q8_0":
            tensors.append((name, (n_in, n_out), T_Q8_0, lambda: q8_0_bytes(rng, n_out, n_in)))
        elif six:
            tensors.append((name, (n_in, n_out), T_Q6_K, lambda: q6_k_bytes(rng, n_out, n_in)))
        else:
            tensors.append((name, (n_in, n_out), T_Q4_K, lambda: q4_k_bytes(rng, n_out, n_in)))

    def vec(name, n, kind):
        if kind == "norm":
            tensors.append((name, (n,), T_F32, lambda: (1.0 + 0.05 * rng.standard_normal(n)).astype(np.float32)))
        else:
            tensors.append((name, (n,), T_F32, lambda: (0.1 * rng.standard_normal(n)).astype(np.float32)))

    assert quant in ("q8_0", "q4_k_m")
    mat("token_embd.weight", ne, vocab, six=True)
    vec("output_norm.weight", ne, "norm")
    for i in range(cfg["n_layer"]):
        p = "blk.%d." % i
        vec(p + "attn_norm.weight", ne, "norm")
        mat(p + "attn_q.weight", ne, nh * hd)
        mat(p + "attn_k.weight", ne, nkv * hd)
        mat(p + "attn_v.weight", ne, nkv * hd, six=more_bits(i, cfg["n_layer"]))
        mat(p + "attn_output.weight", nh * hd, ne)
        vec(p + "ffn_norm.weight", ne, "norm")
        mat(p + "ffn_gate.weight", ne, nff)
        mat(p + "ffn_up.weight", ne, nff)
        mat(p + "ffn_down.weight", nff, ne, six=more_bits(i, cfg["n_layer"]))
        if cfg["bias"]:
            vec(p + "attn_q.bias", nh * hd, "bias")
            vec(p + "attn_k.bias", nkv * hd, "bias")
            vec(p + "attn_v.bias", nkv * hd, "bias")

    def nbytes(dims, typ):
        n = int(np.prod(dims))
        return n * 4 if typ == T_F32 else n // BLOCK[typ][0] * BLOCK[typ][1]

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
    ap.add_argument("--quant", default="q8_0", choices=["q8_0", "q4_k_m"])
    args = ap.parse_args()
    cfg = dict(ARCHS[args.arch])
    if args.layers:
        cfg["n_layer"] = args.layers
    n = write_model(args.out, cfg, args.seed, quant=args.quant)
    print("wrote %s: %s (%s), %d layers, %.1f MB of tensor data" % (args.out, args.arch, args.quant, cfg["n_layer"], n / 1e6))


if __name__ == "__main__":
    main()
