"""End-to-end drop-in check and timing: the reference's own model code on a synthetic model, linked three ways.

TEST INFRASTRUCTURE (see oracle/e2e/driver.cpp, oracle/Makefile target e2e).  Needs the binaries under oracle/_ref/
(built where the reference tree is present) and a B200.

    python oracle/e2e/run_e2e.py --arch qwen2-1.5b --prompt 45 --gen 128 --ctx 4096 --batch 512 [--cpu] [--zerocopy]

Runs e2e_ref (the reference's GPU path, weights in device memory) greedily, then e2e_b200 (this repository's
attention kernels dropped into the same model code; once call by call, once with OATTN_FUSE_CALL_SEQUENCE=1) on the
same token sequence, and reports for each build TTFT and
TPOT, and between builds the step-by-step top-1 agreement and the largest logit difference after the prompt and after
the last step.  --cpu adds the reference's CPU build as the fp32 oracle of the whole model (slow: use --arch tiny);
--zerocopy adds the reference's GPU path exactly as it is (weights read through a host mapping).
Prints one JSON object.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REFDIR = os.path.join(os.path.dirname(HERE), "_ref")
sys.path.insert(0, HERE)
import make_gguf  # noqa: E402


def binaries():
    return {n: os.path.join(REFDIR, n) for n in ("e2e_cpu", "e2e_ref", "e2e_ref_zerocopy", "e2e_b200", "e2e_b200_placed")}


def available():
    b = binaries()
    return all(os.path.exists(b[n]) for n in ("e2e_ref", "e2e_b200"))


def run_build(exe, model, tmp, tag, args, force=None, env=None):
    tok, lg = os.path.join(tmp, tag + "_tok.bin"), os.path.join(tmp, tag + "_logits.bin")
    cmd = [exe, "--model", model, "--prompt", str(args.prompt), "--gen", str(args.gen), "--ctx", str(args.ctx),
           "--batch", str(args.batch), "--seed", str(args.seed), "--tokens-out", tok, "--logits-out", lg]
    if not args.no_warmup:
        cmd.append("--warmup")
    if force:
        cmd += ["--force", force]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=args.timeout, env=dict(os.environ, **(env or {})))
    if p.returncode != 0:
        raise RuntimeError("%s failed (%d): %s" % (tag, p.returncode, (p.stderr or p.stdout)[-800:]))
    line = [x for x in p.stdout.splitlines() if x.startswith("{")][-1]
    r = json.loads(line)
    r["tokens"] = np.fromfile(tok, np.int32)
    r["logits"] = np.fromfile(lg, np.float32).reshape(2, -1)
    return r


def compare(a, b):
    n = min(len(a["tokens"]), len(b["tokens"]))
    d = np.abs(a["logits"] - b["logits"])
    return {"top1_agreement": float((a["tokens"][:n] == b["tokens"][:n]).mean()), "steps_compared": int(n),
            "max_logit_diff_after_prompt": float(d[0].max()), "max_logit_diff_after_last_step": float(d[1].max()),
            "logit_scale": float(np.abs(a["logits"]).max())}


def against_golden(r, gold):
    """A GPU build that was fed the CPU oracle's tokens: where does its own top-1 agree with the oracle's, and how
    large was the oracle's top-1 - top-2 margin where it does not."""
    n = min(len(r["tokens"]), len(gold["tokens"]))
    same = r["tokens"][:n] == gold["tokens"][:n]
    margin = gold["top2"][:n, 0] - gold["top2"][:n, 1]
    idx, val = gold["head_idx"], gold["head_val"]
    d = np.abs(np.take_along_axis(r["logits"], idx, axis=1) - val)
    return {"top1_agreement": float(same.mean()), "points_compared": int(n),
            "oracle_margin_median": float(np.median(margin)),
            "oracle_margin_at_disagreements": [float(x) for x in margin[~same]],
            "max_logit_diff_on_oracle_top64_after_prompt": float(d[0].max()),
            "max_logit_diff_on_oracle_top64_after_last_step": float(d[1].max()),
            "logit_scale": float(np.abs(val).max())}


def run_golden(config, timeout=1800, model=None):
    """An end-to-end configuration whose CPU-oracle run is stored in tests/golden/e2e_<config>_cpu.npz
    (tests/golden/make_e2e_golden.py): writes the same synthetic model, runs the reference's GPU build and the drop-in
    (call by call, and with call-sequence fusion) on the oracle's token sequence, and compares their top-1 choices and
    logits with the oracle's.  Returns a dict with TTFT / TPOT of every build as well."""
    gpath = os.path.join(os.path.dirname(os.path.dirname(HERE)), "tests", "golden", "e2e_%s_cpu.npz" % config)
    g = np.load(gpath)
    cfg = json.loads(str(g["params"]))
    gold = {k: g[k] for k in ("tokens", "top2", "head_idx", "head_val")}
    args = parser().parse_args(["--arch", cfg["arch"], "--prompt", str(cfg["prompt"]), "--gen", str(cfg["gen"]), "--ctx",
                                str(cfg["ctx"]), "--batch", str(cfg["batch"]), "--seed", str(cfg["seed"]), "--timeout", str(timeout)])
    exe = binaries()
    out = {"config": config, **cfg, "oracle_run": json.loads(str(g["run"]))}
    with tempfile.TemporaryDirectory() as tmp:
        if model is None:
            model = os.path.join(tmp, "model.gguf")
            make_gguf.write_model(model, dict(make_gguf.ARCHS[cfg["arch"]]), seed=cfg["model_seed"], quant=cfg["quant"])
        forced = os.path.join(tmp, "forced.bin")
        gold["tokens"][:cfg["gen"]].astype(np.int32).tofile(forced)
        builds = {"reference_gpu": (exe["e2e_ref"], None),
                  "b200_dropin": (exe["e2e_b200_placed"] if os.path.exists(exe["e2e_b200_placed"]) else exe["e2e_b200"], None),
                  "b200_dropin_fused_sequence": (exe["e2e_b200"], {"OATTN_FUSE_CALL_SEQUENCE": "1"})}
        for name, (binary, env) in builds.items():
            r = run_build(binary, model, tmp, name, args, forced, env=env)
            out[name] = {**timing(r), "vs_cpu_oracle": against_golden(r, gold)}
    return out


def timing(r):
    return {k: r[k] for k in ("ttft_ms", "tpot_ms", "tpot_ms_after_first", "n_ctx")}


def run(args):
    exe = binaries()
    out = {"arch": args.arch, "quant": args.quant, "layers": args.layers, "prompt": args.prompt, "gen": args.gen, "batch": args.batch}
    with tempfile.TemporaryDirectory() as tmp:
        model = os.path.join(tmp, "model.gguf")
        cfg = dict(make_gguf.ARCHS[args.arch])
        if args.layers:
            cfg["n_layer"] = args.layers
        make_gguf.write_model(model, cfg, seed=args.model_seed, quant=args.quant)
        ref = run_build(exe["e2e_ref"], model, tmp, "ref", args)
        forced = os.path.join(tmp, "forced.bin")
        ref["tokens"][:args.gen].astype(np.int32).tofile(forced)
        b200 = run_build(exe["e2e_b200"], model, tmp, "b200", args, forced)
        # the same binary with call-sequence fusion on: the four calls per layer run as the fused launches
        fused = run_build(exe["e2e_b200"], model, tmp, "b200f", args, forced, env={"OATTN_FUSE_CALL_SEQUENCE": "1"})
        if args.overlap is not None:
            ov = run_build(exe["e2e_b200"], model, tmp, "b200o", args, forced,
                           env={"OATTN_FUSE_CALL_SEQUENCE": "1", "OATTN_DECODE_OVERLAP": str(args.overlap)})
            out["b200_dropin_fused_sequence_overlap%d" % args.overlap] = timing(ov)
        if os.path.exists(exe["e2e_b200_placed"]):
            # the same drop-in with the memory placement done in the source of model_gpu.cu (orin_llm_b200/host/placement.h)
            # instead of by the test-only interposer: must give the same logits, bit for bit
            placed = run_build(exe["e2e_b200_placed"], model, tmp, "b200p", args, forced)
            out["b200_dropin_source_level_placement"] = timing(placed)
            out["source_level_placement_vs_interposed"] = {
                "logits_identical": bool(np.array_equal(placed["logits"], b200["logits"])),
                "tokens_identical": bool(np.array_equal(placed["tokens"], b200["tokens"]))}
        out["reference_gpu"] = timing(ref)
        out["b200_dropin"] = timing(b200)
        out["b200_dropin_fused_sequence"] = timing(fused)
        out["b200_vs_reference_gpu"] = compare(b200, ref)
        out["b200_fused_sequence_vs_reference_gpu"] = compare(fused, ref)
        if args.zerocopy and os.path.exists(exe["e2e_ref_zerocopy"]):
            try:
                out["reference_gpu_zerocopy"] = timing(run_build(exe["e2e_ref_zerocopy"], model, tmp, "zc", args, forced))
            except RuntimeError as e:       # e.g. the host mapping of the weight file is refused on this platform
                out["reference_gpu_zerocopy"] = {"unavailable": str(e)[-300:]}
        if args.cpu and os.path.exists(exe["e2e_cpu"]):
            cpu = run_build(exe["e2e_cpu"], model, tmp, "cpu", args, forced)
            out["reference_cpu"] = timing(cpu)
            out["b200_vs_reference_cpu"] = compare(b200, cpu)
            out["reference_gpu_vs_reference_cpu"] = compare(ref, cpu)
    return out


def parser():
    ap = argparse.ArgumentParser()
    ap.add_argument("--arch", default="tiny", choices=sorted(make_gguf.ARCHS))
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--prompt", type=int, default=45)
    ap.add_argument("--gen", type=int, default=32)
    ap.add_argument("--ctx", type=int, default=4096)
    ap.add_argument("--batch", type=int, default=512)
    ap.add_argument("--seed", type=int, default=7)
    ap.add_argument("--model-seed", type=int, default=1234)
    ap.add_argument("--quant", default="q8_0", choices=["q8_0", "q4_k_m"])
    ap.add_argument("--golden", default=None, choices=["cfg1", "cfg5"],
                    help="run the configuration whose CPU-oracle run is stored under tests/golden/ and compare with it")
    ap.add_argument("--cpu", action="store_true")
    ap.add_argument("--zerocopy", action="store_true")
    ap.add_argument("--no-warmup", action="store_true")
    ap.add_argument("--overlap", type=int, default=None, choices=[0, 1, 2],
                    help="also run the fused-sequence build with this decode launch ordering (OATTN_DECODE_OVERLAP)")
    ap.add_argument("--timeout", type=int, default=900)
    return ap


if __name__ == "__main__":
    _a = parser().parse_args()
    print(json.dumps(run_golden(_a.golden, _a.timeout) if _a.golden else run(_a)))
