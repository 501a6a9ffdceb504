// TEST INFRASTRUCTURE: runs the reference's own Model (src/model.h) on a GGUF file with seeded token ids and prints
// one JSON line.  The same source is linked three ways (oracle/Makefile):
//   e2e_cpu    reference model_cpu.cpp                                  -> the fp32 oracle of the whole model
//   e2e_ref    reference model_gpu.cu + kernels.cu, compiled for sm_100a -> the reference's GPU path as it is
//   e2e_b200   reference model_gpu.cu (unmodified) + kernels.cu with its attention-path wrappers renamed out of the
//              way + this repository's libraries                         -> the drop-in under test
// Protocol: prompt of P seeded token ids through forward_batch in chunks of `batch` (src/engine.cpp does the same),
// then G single-token steps.  With --force FILE the token fed at each step comes from FILE (teacher forcing), so that
// several builds can be compared step by step even after their greedy choices diverge; the build's own argmax is
// still recorded.  --warmup runs an untimed pass first, so that one-time costs stay out of TTFT and TPOT.
// --top2-out FILE writes, for the point after the prompt and after every step, the two largest logits (the margin that
// says how much a top-1 disagreement means).
// Built with -DE2E_ATTN_HOOK against the CPU model source with two hook calls inserted (oracle/Makefile, target
// e2e_cpu_dump; the arithmetic is untouched), --attn-out FILE records what every layer's attention consumed and produced:
// for every token k and v before RoPE, and from position --attn-from on also q before RoPE, q and k after it and the
// attention output.  Record = int32 {stage, layer, n_past, nq, nkv} + floats: stage 0 -> q[nq] k[nkv] v[nkv];
// stage 1 -> q_rot[nq] k_rot[nkv] attn[nq]  (nq = 0: k and v only).
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "gguf.h"
#include "model.h"

#ifdef E2E_ATTN_HOOK
static FILE* g_attn_f = nullptr;
static int g_attn_from = 0;
extern "C" void e2e_attn_hook(int stage, int layer, int n_past, const float* q, const float* k, const float* v,
                              const float* attn, int nq, int nkv) {
    if (!g_attn_f) return;
    const bool full = n_past >= g_attn_from;
    if (stage == 1 && !full) return;
    const int32_t head[5] = {stage, layer, n_past, full ? nq : 0, nkv};
    fwrite(head, sizeof(int32_t), 5, g_attn_f);
    if (full) fwrite(q, sizeof(float), nq, g_attn_f);
    fwrite(k, sizeof(float), nkv, g_attn_f);
    if (stage == 0) fwrite(v, sizeof(float), nkv, g_attn_f);
    else fwrite(attn, sizeof(float), nq, g_attn_f);
}
#endif

static double now_ms() {
    return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

static void top2(const float* x, int n, float* out) {
    float a = -1e30f, b = -1e30f;
    for (int i = 0; i < n; ++i) {
        if (x[i] > a) { b = a; a = x[i]; }
        else if (x[i] > b) b = x[i];
    }
    out[0] = a;
    out[1] = b;
}

static int argmax(const float* x, int n) {
    int best = 0;
    for (int i = 1; i < n; ++i)
        if (x[i] > x[best]) best = i;
    return best;
}

int main(int argc, char** argv) {
    std::string path, force, tokens_out, logits_out, top2_out, attn_out;
    int attn_from = 0;
    int n_prompt = 45, n_gen = 16, n_ctx = 4096, batch = 512;
    uint64_t seed = 7;
    bool warmup = false;
    for (int i = 1; i < argc; ++i) {
        std::string a = argv[i];
        auto next = [&]() { return std::string(i + 1 < argc ? argv[++i] : ""); };
        if (a == "--model") path = next();
        else if (a == "--prompt") n_prompt = atoi(next().c_str());
        else if (a == "--gen") n_gen = atoi(next().c_str());
        else if (a == "--ctx") n_ctx = atoi(next().c_str());
        else if (a == "--batch") batch = atoi(next().c_str());
        else if (a == "--seed") seed = strtoull(next().c_str(), nullptr, 10);
        else if (a == "--force") force = next();
        else if (a == "--warmup") warmup = true;
        else if (a == "--tokens-out") tokens_out = next();
        else if (a == "--logits-out") logits_out = next();
        else if (a == "--top2-out") top2_out = next();
        else if (a == "--attn-out") attn_out = next();
        else if (a == "--attn-from") attn_from = atoi(next().c_str());
        else { fprintf(stderr, "unknown argument %s\n", a.c_str()); return 2; }
    }
    if (path.empty()) { fprintf(stderr, "usage: driver --model file.gguf [--prompt P --gen G --ctx C --batch B]\n"); return 2; }

    llm::GGUF gguf;
    gguf.load(path);
    llm::Model model;
    model.load(gguf);
    model.init_buffers(n_ctx, batch);
    const int n_vocab = model.hparams.n_vocab;

    std::vector<int32_t> prompt(n_prompt);
    uint64_t s = seed * 6364136223846793005ull + 1442695040888963407ull;
    for (int i = 0; i < n_prompt; ++i) {
        s = s * 6364136223846793005ull + 1442695040888963407ull;
        prompt[i] = (int32_t)((s >> 33) % (uint64_t)n_vocab);
    }
    std::vector<int32_t> forced;
    if (!force.empty()) {
        FILE* f = fopen(force.c_str(), "rb");
        if (!f) { fprintf(stderr, "cannot open %s\n", force.c_str()); return 2; }
        int32_t t;
        while (fread(&t, sizeof(t), 1, f) == 1) forced.push_back(t);
        fclose(f);
    }

    // Untimed pass over the first chunk and one single-token step: module loading, first-use initialisation and (GPU
    // builds) the capture of the decode graph happen here, for every build alike.  The timed run starts again at
    // position 0 and overwrites what this wrote.
    if (warmup) {
        const int n = std::min(batch, n_prompt);
        if (n > 1) model.forward_batch(prompt.data(), n, 0);
        model.forward(prompt[0], n > 1 ? n : 0);
    }

#ifdef E2E_ATTN_HOOK
    if (!attn_out.empty()) {
        g_attn_f = fopen(attn_out.c_str(), "wb");
        g_attn_from = attn_from;
    }
#else
    (void)attn_from;
    if (!attn_out.empty()) { fprintf(stderr, "--attn-out needs the build with the attention hooks (e2e_cpu_dump)\n"); return 2; }
#endif
    std::vector<float> margins;               // top-1 and top-2 logit after the prompt and after every step

    // prefill
    const double t0 = now_ms();
    const float* logits = nullptr;
    for (int done = 0; done < n_prompt; done += batch) {
        const int n = std::min(batch, n_prompt - done);
        logits = n == 1 ? model.forward(prompt[done], done) : model.forward_batch(prompt.data() + done, n, done);
    }
    const double ttft = now_ms() - t0;
    std::vector<float> first_logits(logits, logits + n_vocab);
    std::vector<int32_t> own;                 // this build's argmax after the prompt and after every step
    own.push_back(argmax(logits, n_vocab));
    margins.resize(2);
    top2(logits, n_vocab, margins.data());

    // decode
    std::vector<double> step_ms;
    int n_past = n_prompt;
    for (int g = 0; g < n_gen; ++g) {
        const int32_t tok = g < (int)forced.size() ? forced[g] : own.back();
        const double t1 = now_ms();
        logits = model.forward(tok, n_past++);
        step_ms.push_back(now_ms() - t1);
        own.push_back(argmax(logits, n_vocab));
        margins.resize(margins.size() + 2);
        top2(logits, n_vocab, margins.data() + margins.size() - 2);
    }
#ifdef E2E_ATTN_HOOK
    if (g_attn_f) { fclose(g_attn_f); g_attn_f = nullptr; }
#endif
    if (!top2_out.empty()) {
        FILE* f = fopen(top2_out.c_str(), "wb");
        fwrite(margins.data(), sizeof(float), margins.size(), f);
        fclose(f);
    }
    double tpot = 0.0, tpot_rest = 0.0;
    for (size_t i = 0; i < step_ms.size(); ++i) {
        tpot += step_ms[i];
        if (i > 0) tpot_rest += step_ms[i];      // the first step includes graph capture in the GPU builds
    }
    if (!tokens_out.empty()) {
        FILE* f = fopen(tokens_out.c_str(), "wb");
        fwrite(own.data(), sizeof(int32_t), own.size(), f);
        fclose(f);
    }
    if (!logits_out.empty()) {
        FILE* f = fopen(logits_out.c_str(), "wb");
        fwrite(first_logits.data(), sizeof(float), n_vocab, f);
        fwrite(logits, sizeof(float), n_vocab, f);
        fclose(f);
    }
    printf("{\"n_prompt\": %d, \"n_gen\": %d, \"n_ctx\": %d, \"batch\": %d, \"ttft_ms\": %.3f, \"tpot_ms\": %.4f, "
           "\"tpot_ms_after_first\": %.4f, \"first_token\": %d, \"last_token\": %d}\n",
           n_prompt, n_gen, model.hparams.n_ctx, batch, ttft, step_ms.empty() ? 0.0 : tpot / step_ms.size(),
           step_ms.size() > 1 ? tpot_rest / (step_ms.size() - 1) : 0.0, own.front(), own.back());
    return 0;
}
