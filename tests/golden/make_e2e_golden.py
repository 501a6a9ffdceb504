"""Generates tests/golden/e2e_<config>_cpu.npz: what the reference's CPU build (the fp32 oracle of the whole model) does on
an end-to-end configuration, in a form small enough to commit.

TEST INFRASTRUCTURE.  Runs oracle/_ref/e2e_cpu (the reference's own model_cpu.cpp behind oracle/e2e/driver.cpp, built
by `make -C oracle e2e REF=<reference checkout>`) on the synthetic model of oracle/e2e/make_gguf.py, greedy and
free-running, and keeps
    tokens   the oracle's top-1 token after the prompt and after every decode step  (int32, 1 + gen)
    top2     its two largest logits at each of those points                           (fp32, [1 + gen][2])
    head_idx, head_val   the 64 largest logits after the prompt and after the last step (indices and values)
together with the parameters that reproduce the run (architecture, quantisation, seeds, prompt length, context, chunk).
The GPU tests feed `tokens` to the GPU builds (teacher forcing) and compare their top-1 choices with it.

    python tests/golden/make_e2e_golden.py --config cfg1      # Qwen2.5-1.5B shape, Q8_0, 45 + 128 tokens   (~5 min)
    python tests/golden/make_e2e_golden.py --config cfg5      # Llama-3-8B shape, Q4_K_M mix, 512 + 128     (~80 min)
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "oracle", "e2e"))
import make_gguf  # noqa: E402

CONFIGS = {
    "cfg1": dict(arch="qwen2-1.5b", quant="q8_0", prompt=45, gen=128, ctx=4096, batch=512, seed=7, model_seed=1234),
    "cfg5": dict(arch="llama3-8b", quant="q4_k_m", prompt=512, gen=128, ctx=8192, batch=512, seed=7, model_seed=1234),
}


def pack(cfg, line, tokens, top2, logits):
    order = np.argsort(-logits, axis=1)[:, :64]
    return dict(tokens=tokens.astype(np.int32), top2=top2.reshape(-1, 2).astype(np.float32),
                head_idx=order.astype(np.int32), head_val=np.take_along_axis(logits, order, axis=1).astype(np.float32),
                params=np.array(json.dumps(cfg)), run=np.array(json.dumps(line)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True, choices=sorted(CONFIGS))
    ap.add_argument("--from-dir", default=None, help="pack the output files of a run made by hand (<config>_tok.bin, ...)")
    ap.add_argument("--model", default=None, help="reuse a model file written earlier with the same parameters")
    args = ap.parse_args()
    cfg = CONFIGS[args.config]
    out = os.path.join(HERE, "e2e_%s_cpu.npz" % args.config)
    with tempfile.TemporaryDirectory() as tmp:
        d = args.from_dir or tmp
        pre = os.path.join(d, args.config)
        if not args.from_dir:
            exe = os.path.join(ROOT, "oracle", "_ref", "e2e_cpu")
            model = args.model or os.path.join(tmp, "model.gguf")
            if not args.model:
                make_gguf.write_model(model, dict(make_gguf.ARCHS[cfg["arch"]]), seed=cfg["model_seed"], quant=cfg["quant"])
            with open(pre + ".json", "w") as f:
                subprocess.check_call([exe, "--model", model, "--prompt", str(cfg["prompt"]), "--gen", str(cfg["gen"]), "--ctx",
                                       str(cfg["ctx"]), "--batch", str(cfg["batch"]), "--seed", str(cfg["seed"]), "--tokens-out",
                                       pre + "_tok.bin", "--logits-out", pre + "_logits.bin", "--top2-out", pre + "_top2.bin"],
                                      stdout=f)
        line = json.loads([x for x in open(pre + ".json") if x.startswith("{")][-1])
        tokens = np.fromfile(pre + "_tok.bin", np.int32)
        top2 = np.fromfile(pre + "_top2.bin", np.float32)
        logits = np.fromfile(pre + "_logits.bin", np.float32).reshape(2, -1)
        assert len(tokens) == cfg["gen"] + 1 and len(top2) == 2 * (cfg["gen"] + 1)
        np.savez_compressed(out, **pack(cfg, line, tokens, top2, logits))
    print("wrote", out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
    main()
