"""Generates tests/golden/*.npz from the REFERENCE's own CPU code (oracle/_ref/libref_attn.so).

Run where the reference tree is present:   python tests/golden/make_golden.py
The fixtures are what pins oracle/attn_oracle.c (and, through it, the CUDA path) to the
reference: each case stores the inputs that the reference's unmodified forward() fed to its
attention block and the outputs it produced.  The reference ships no golden vectors itself.

Cases (all tiny; fp32):
  probe_neox    qwen-style neox RoPE, 6 q heads / 2 kv heads, d=64,  n_rot=64, theta=1e6, 9 tokens
  probe_normal  llama-style normal RoPE, 8/2 heads, d=128, n_rot=128, theta=5e5, freq factors, 7 tokens
  probe_partial normal RoPE with n_rot=32 < d=64 (partial rotation), 4/4 heads, 5 tokens
  kvshift       the reference's kv_shift on a random fp32 cache
  probe_pre_qwen2  as probe_neox plus q/k/v biases (Qwen2.5-style layer), 6/2 heads, d=128, 8 tokens
  probe_pre_qwen3  neox RoPE plus per-head q/k RMSNorm weights and biases together, 8/2 heads, d=128, eps 1e-6, 8 tokens

python tests/golden/make_golden.py [case ...] regenerates only the named cases (default: all).
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle.oracle import RefLib  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


def probe(ref, name, seed, n_tok, n_head, n_kv, d, rope_type, n_rot, theta, with_ff):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((n_tok, n_head * d)).astype(np.float32)
    ff = None
    if with_ff:
        ff = (1.0 + rng.random(n_rot // 2) * 7.0).astype(np.float32)
    n_ctx = 16
    r = ref.forward_probe(x, n_head, n_kv, d, n_ctx, rope_type, n_rot, theta, ff)
    np.savez_compressed(
        os.path.join(OUT, name + ".npz"), x=x, n_head=n_head, n_kv=n_kv, d=d, n_ctx=n_ctx,
        rope_type=rope_type, n_rot=n_rot, theta=np.float32(theta),
        freq_factors=ff if ff is not None else np.zeros(0, np.float32), **r)
    print(name, "ok", {k: v.shape for k, v in r.items()})


def probe_pre(ref, name, seed, n_tok, n_head, n_kv, d, rope_type, theta, with_bias, with_norm, eps):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((n_tok, n_head * d)).astype(np.float32)
    z = np.zeros(0, np.float32)
    bq = (0.5 * rng.standard_normal(n_head * d)).astype(np.float32) if with_bias else None
    bk = (0.5 * rng.standard_normal(n_kv * d)).astype(np.float32) if with_bias else None
    bv = (0.5 * rng.standard_normal(n_kv * d)).astype(np.float32) if with_bias else None
    nq = (1.0 + 0.3 * rng.standard_normal(d)).astype(np.float32) if with_norm else None
    nk = (1.0 + 0.3 * rng.standard_normal(d)).astype(np.float32) if with_norm else None
    n_ctx = 16
    r = ref.forward_probe_pre(x, n_head, n_kv, d, n_ctx, rope_type, d, theta, bq, bk, bv, nq, nk, eps)
    np.savez_compressed(
        os.path.join(OUT, name + ".npz"), x=x, n_head=n_head, n_kv=n_kv, d=d, n_ctx=n_ctx, rope_type=rope_type, n_rot=d,
        theta=np.float32(theta), eps=np.float32(eps),
        bias_q=bq if bq is not None else z, bias_k=bk if bk is not None else z, bias_v=bv if bv is not None else z,
        norm_q=nq if nq is not None else z, norm_k=nk if nk is not None else z, **r)
    print(name, "ok", {k: v.shape for k, v in r.items()})


def main():
    ref = RefLib()
    want = set(sys.argv[1:])

    def on(name):
        return not want or name in want
    if on("probe_neox"):
        probe(ref, "probe_neox", 101, 9, 6, 2, 64, 1, 64, 1e6, False)
    if on("probe_normal"):
        probe(ref, "probe_normal", 102, 7, 8, 2, 128, 0, 128, 5e5, True)
    if on("probe_partial"):
        probe(ref, "probe_partial", 103, 5, 4, 4, 64, 0, 32, 1e4, False)
    if on("probe_pre_qwen2"):
        probe_pre(ref, "probe_pre_qwen2", 105, 8, 6, 2, 128, 1, 1e6, True, False, 1e-6)
    if on("probe_pre_qwen3"):
        probe_pre(ref, "probe_pre_qwen3", 106, 8, 8, 2, 128, 1, 1e6, True, True, 1e-6)
    if not on("kvshift"):
        return

    rng = np.random.default_rng(104)
    n_layer, n_kv, d, n_ctx, n_keep, shift = 2, 3, 8, 12, 2, 5
    k0 = rng.standard_normal((n_layer, n_kv, n_ctx, d)).astype(np.float32)
    v0 = rng.standard_normal((n_layer, n_kv, n_ctx, d)).astype(np.float32)
    k1, v1 = k0.copy(), v0.copy()
    ref.kv_shift(k1, v1, n_layer, n_kv, d, n_ctx, n_keep, shift)
    np.savez_compressed(os.path.join(OUT, "kvshift.npz"), k0=k0, v0=v0, k1=k1, v1=v1, n_keep=n_keep, shift=shift)
    print("kvshift ok")


if __name__ == "__main__":
    main()
