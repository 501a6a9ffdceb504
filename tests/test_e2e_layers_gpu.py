"""End-to-end configurations against the reference's CPU build (the fp32 oracle of the whole model), full model shapes.

1. Per-layer attention, teacher-forced: the CPU build (with two hook calls inserted into a build-time copy of its model
   source; no arithmetic changed) records what every layer's attention consumed and produced on the Qwen2.5-1.5B shape.
   Each layer's q / k / v are fed to this repository's fused prefill and decode calls and the attention outputs are
   compared layer by layer: max-abs <= 1e-2, mean-abs <= 1e-3.  This is the pass/fail of the end-to-end check, because it
   isolates attention from the int8 activation quantisation of the GEMVs around it.
2. Free-running comparison beside it: the reference's GPU build and the drop-in are fed the CPU oracle's greedy token
   sequence (stored in tests/golden/e2e_<config>_cpu.npz) and their top-1 choices are compared with the oracle's, with
   the oracle's top-1 - top-2 margin at every disagreement.

The binaries under oracle/_ref/ are test infrastructure built where the reference tree is present; tests skip without
them."""
import os
import struct
import subprocess
import sys

import numpy as np
import pytest
import torch

from helpers import MAX_ABS_TOL, MEAN_ABS_TOL

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "oracle", "e2e"))
DUMP_EXE = os.path.join(ROOT, "oracle", "_ref", "e2e_cpu_dump")


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.fixture(scope="module")
def qwen_model(tmp_path_factory):
    import make_gguf
    path = str(tmp_path_factory.mktemp("e2e") / "qwen2-1.5b.gguf")
    make_gguf.write_model(path, dict(make_gguf.ARCHS["qwen2-1.5b"]), seed=1234, quant="q8_0")
    return path


def read_records(path):
    """{(stage, layer, n_past): dict of arrays} from the dump file (format: oracle/e2e/driver.cpp)."""
    rec = {}
    b = open(path, "rb").read()
    off = 0
    while off < len(b):
        stage, layer, n_past, nq, nkv = struct.unpack_from("<5i", b, off)
        off += 20

        def take(n):
            nonlocal off
            a = np.frombuffer(b, np.float32, n, off).copy()
            off += 4 * n
            return a
        q = take(nq)
        k = take(nkv)
        last = take(nkv if stage == 0 else nq)
        rec[(stage, layer, n_past)] = {"q": q, "k": k, "v" if stage == 0 else "attn": last}
    return rec


def test_per_layer_attention_teacher_forced(ops, oracle, qwen_model, tmp_path):
    if not os.path.exists(DUMP_EXE):
        pytest.skip("oracle/_ref/e2e_cpu_dump not built (needs the reference tree at build time)")
    n_prompt, n_gen, first = 45, 4, 40          # q and outputs recorded from position 40 on; k, v for every position
    dump = str(tmp_path / "attn.bin")
    p = subprocess.run([DUMP_EXE, "--model", qwen_model, "--prompt", str(n_prompt), "--gen", str(n_gen), "--ctx", "4096",
                        "--batch", "512", "--seed", "7", "--attn-out", dump, "--attn-from", str(first)],
                       capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-500:]
    rec = read_records(dump)
    n_layer, n_head, n_kv, hd, n_ctx = 28, 12, 2, 128, 256
    n_tok = n_prompt + n_gen
    scale = float(1.0 / np.sqrt(hd))
    rope = (ops.ROPE_NEOX, hd, 1e6, None)
    worst = (0.0, 0.0, -1)
    for l in range(n_layer):
        k_pre = np.stack([rec[(0, l, t)]["k"] for t in range(n_tok)]).reshape(n_tok, n_kv, hd)
        v_pre = np.stack([rec[(0, l, t)]["v"] for t in range(n_tok)]).reshape(n_tok, n_kv, hd)
        q_pre = np.stack([rec[(0, l, t)]["q"] for t in range(first, n_tok)]).reshape(-1, n_head, hd)
        want = np.stack([rec[(1, l, t)]["attn"] for t in range(first, n_tok)]).reshape(-1, n_head, hd)
        # history rows 0..first-1: rotated by the oracle's RoPE (the CPU backend's arithmetic), rounded to fp16 like the cache
        kc = np.zeros((n_kv, n_ctx, hd), np.float16)
        vc = np.zeros((n_kv, n_ctx, hd), np.float16)
        for t in range(first):
            kr = k_pre[t].copy()
            for h in range(n_kv):
                oracle.rope(kr[h], 1, hd, 1e6, t)
            kc[:, t] = kr.astype(np.float16)
            vc[:, t] = v_pre[t].astype(np.float16)
        dK, dV = dev(kc), dev(vc)
        out = torch.empty(n_tok - first, n_head, hd, device="cuda")
        nb = n_prompt - first
        # the tail of the prompt as one fused prefill chunk, then the decode steps one by one, as the engine runs them
        ops.attn_prefill(dev(q_pre[:nb]), dev(k_pre[first:n_prompt]), dev(v_pre[first:n_prompt]), dK, dV, out[:nb], n_head, n_kv,
                         hd, n_ctx, first, nb, scale, ops.FUSE_ALL, rope)
        d_pos = torch.zeros(1, dtype=torch.int32, device="cuda")
        for t in range(n_prompt, n_tok):
            d_pos.fill_(t)
            ops.attn_decode(dev(q_pre[t - first]), dev(k_pre[t]), dev(v_pre[t]), dK, dV, out[t - first], n_head, n_kv, hd, n_ctx,
                            d_pos, scale, ops.FUSE_ALL, rope)
        torch.cuda.synchronize()
        err = np.abs(out.cpu().numpy() - want)
        assert np.isfinite(err).all()
        mx, mean = float(err.max()), float(err.mean())
        assert mx <= MAX_ABS_TOL and mean <= MEAN_ABS_TOL, "layer %d: max-abs %.3e mean-abs %.3e" % (l, mx, mean)
        if mx > worst[0]:
            worst = (mx, mean, l)
        # the appended K rows are the oracle's rotated k, to fp16 rounding
        k_rot = np.stack([rec[(1, l, t)]["k"] for t in range(first, n_tok)]).reshape(-1, n_kv, hd)
        got = dK[:, first:n_tok].float().cpu().numpy().transpose(1, 0, 2)
        assert np.abs(got - k_rot).max() <= 2.0 ** -9 * max(1.0, float(np.abs(k_rot).max())), "layer %d appended K" % l
    print("per-layer teacher-forced attention, %d layers: worst max-abs %.2e (mean-abs %.2e) at layer %d" % (
        n_layer, worst[0], worst[1], worst[2]))


@pytest.mark.parametrize("config", ["cfg1", "cfg5"])
def test_top1_agreement_with_the_cpu_oracle(config, qwen_model):
    import run_e2e
    gold = os.path.join(ROOT, "tests", "golden", "e2e_%s_cpu.npz" % config)
    if not run_e2e.available() or not os.path.exists(gold):
        pytest.skip("oracle/_ref/e2e_* or the stored oracle run is missing")
    if config == "cfg5" and os.environ.get("OATTN_SKIP_8B"):
        pytest.skip("OATTN_SKIP_8B is set")
    r = run_e2e.run_golden(config, model=qwen_model if config == "cfg1" else None)
    ref, b200, fused = (r[n]["vs_cpu_oracle"] for n in ("reference_gpu", "b200_dropin", "b200_dropin_fused_sequence"))
    print(config, {n: (r[n]["vs_cpu_oracle"]["top1_agreement"], r[n]["ttft_ms"], r[n]["tpot_ms_after_first"])
                   for n in ("reference_gpu", "b200_dropin", "b200_dropin_fused_sequence")})
    for c in (b200, fused):
        # Random-init logits are nearly tied and both GPU builds quantise activations to int8 for every GEMV / GEMM, so
        # top-1 flips for reasons that have nothing to do with attention (on the Q4_K_M model the reference's own GPU build
        # agrees with its CPU build on little more than half of the steps): the bar is the reference's own GPU build.
        assert c["top1_agreement"] >= ref["top1_agreement"] - 0.07, (c, ref)
        assert c["max_logit_diff_on_oracle_top64_after_last_step"] <= \
            1.5 * ref["max_logit_diff_on_oracle_top64_after_last_step"] + 0.02 * c["logit_scale"], (c, ref)
        # the disagreements sit where the oracle itself was nearly undecided
        miss = c["oracle_margin_at_disagreements"]
        if miss:
            assert float(np.median(miss)) <= 1.25 * c["oracle_margin_median"], c
