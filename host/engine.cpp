// engine.cpp - the C++ host of the B200 kernels: `engine gen <token ids>` as the reference's engine offers it
// (ref: src/engine.cu:1276 LK_PACK, :1612-1626 argv tokens + LK_PROMPT_BIN, :1729-1734 batched prefill of all but
// the last prompt token, :1763-1797 decode loop and RESULT line).  Only that path: no profilers, dumps or
// perplexity mode.
//
//   LK_PACK=<pack>  [LK_PROMPT_BIN=<int32 blob>]  [LK_NGEN=n]  [LK_MAX_SEQ=n]  [LK_PF_CHUNK=n]  [LK_BENCH=1]
//       engine gen [token ids ...]
//
// The pack (lfm2-ampere_b200/pack.py) holds every tensor in the planar layout the kernels read; it is copied to the
// device once.  Prompt tokens 0..n-2 run through the batched-prefill call sequence in chunks of LK_PF_CHUNK
// (dense Q4_0 x Q8_1 GEMMs around the chunk kernels, the MoE FFN as count / plan / scatter + two grouped GEMMs);
// the last prompt token and every generated token run through the decode step, captured once in a CUDA graph
// whose inputs (token id, position) live on the device and are advanced by the argmax kernel, so a replay needs
// no host argument.  All kernels are reached through the C ABI of include/lkb.h (lkb_shim.hpp's wrappers keep
// the reference's kernel names); this file contains no device code and is compiled by g++.
#include <cuda_runtime_api.h>

#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "lkb_shim.hpp"

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { \
    fprintf(stderr, "CUDA error %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, __LINE__); exit(1); } } while (0)

namespace {

constexpr int H = LKB_HIDDEN, E = LKB_N_EXPERTS, TOPK = LKB_TOP_K, I = LKB_MOE_INTER;
constexpr int N_KV = 8, HEAD_DIM = 64, QKV = H + 2 * N_KV * HEAD_DIM, CONV_ROWS = 3 * H, BPR = H / 32, SBPR = H / 256;
constexpr float EPS = 1e-5f;

struct Pack {
    unsigned n_layers = 0, vocab = 0;
    float theta = 0.0f;
    unsigned char * dev = nullptr;
    std::map<std::string, std::pair<uint64_t, uint64_t>> tab;
    const void * at(const std::string & name) const {
        auto it = tab.find(name);
        if (it == tab.end()) { fprintf(stderr, "pack: tensor %s missing\n", name.c_str()); exit(1); }
        return dev + it->second.first;
    }
    bool has(const std::string & name) const { return tab.count(name) != 0; }
    const float * f32(const std::string & name) const { return static_cast<const float *>(at(name)); }
};

Pack load_pack(const char * path) {
    FILE * f = fopen(path, "rb");
    if (!f) { fprintf(stderr, "LK_PACK: cannot open %s\n", path); exit(1); }
    unsigned char head[32];
    if (fread(head, 1, 32, f) != 32 || memcmp(head, "LKBPACK1", 8) != 0) { fprintf(stderr, "LK_PACK: %s is not an LKBPACK1 file\n", path); exit(1); }
    Pack p;
    unsigned n_tensors;
    memcpy(&p.n_layers, head + 8, 4); memcpy(&p.vocab, head + 12, 4); memcpy(&p.theta, head + 16, 4); memcpy(&n_tensors, head + 20, 4);
    for (unsigned i = 0; i < n_tensors; ++i) {
        unsigned char e[64];
        if (fread(e, 1, 64, f) != 64) { fprintf(stderr, "LK_PACK: truncated table\n"); exit(1); }
        e[47] = 0;
        uint64_t off, nb;
        memcpy(&off, e + 48, 8); memcpy(&nb, e + 56, 8);
        p.tab[reinterpret_cast<const char *>(e)] = {off, nb};
    }
    if (fseek(f, 0, SEEK_END) != 0) { fprintf(stderr, "LK_PACK: seek\n"); exit(1); }
    const long total = ftell(f);
    for (auto & kv : p.tab)
        if ((long) (kv.second.first + kv.second.second) > total) { fprintf(stderr, "LK_PACK: tensor %s runs past the file\n", kv.first.c_str()); exit(1); }
    void * base;
    CK(cudaMalloc(&base, (size_t) total));
    p.dev = static_cast<unsigned char *>(base);
    // staged through one pinned buffer: the file is read once, in 64 MB pieces
    const size_t piece = (size_t) 64 << 20;
    void * stage_v;
    CK(cudaMallocHost(&stage_v, piece));
    unsigned char * stage = static_cast<unsigned char *>(stage_v);
    rewind(f);
    for (size_t done = 0; done < (size_t) total;) {
        const size_t n = fread(stage, 1, piece, f);
        if (n == 0) { fprintf(stderr, "LK_PACK: read\n"); exit(1); }
        CK(cudaMemcpy(p.dev + done, stage, n, cudaMemcpyHostToDevice));
        done += n;
    }
    CK(cudaFreeHost(stage));
    fclose(f);
    return p;
}

template <typename T> T * dalloc(size_t n) {
    void * p;
    CK(cudaMalloc(&p, n * sizeof(T)));
    CK(cudaMemset(p, 0, n * sizeof(T)));
    return static_cast<T *>(p);
}

struct MixerW {
    bool is_attn;
    const float * attn_norm;
    lk::QT4 in_proj, out, wq, wk, wv;
    const float * conv_w, * qnorm, * knorm;
    float * hist; void * kc; void * vc;
};

struct Engine {
    Pack pk;
    int n = 0, vocab = 0, max_seq = 0;
    float theta = 0.0f;
    std::vector<MixerW> mx;
    std::vector<lkb_moe_layer> moe;
    const void * eql, * eqh, * esc, * ed;
    const float * out_norm;
    // decode state
    float * x, * ssq, * logits_v, * am_v; int * am_i, * d_token, * d_pos;
    lk::block_q8_1 * xq;
    lkb_moe_layer * moe_dev; lkb_mixer_layer * mixers_dev;
    lkb_moe_scratch scratch; lkb_step_scratch sscratch; lkb_norm_prod_t np_out;
    // prefill chunk state (sized for pf_cap tokens)
    int pf_cap = 0, max_tiles = 0;
    float * X, * a_sc, * inv, * h32, * sel, * sig, * w, * a2_sc, * D, * Y, * o;
    int8_t * a_qs, * a2_qs;
    int * idx, * cnt, * off, * tiles, * ntiles, * perm, * toks;
    void * qh, * gemm_ws; size_t gemm_ws_bytes = 0;
};

lk::QT4 q4(const Pack & p, const std::string & name) { return lk::QT4{p.at(name + ".qs"), p.at(name + ".d")}; }

void build(Engine & e, int max_seq, int pf_cap) {
    const Pack & p = e.pk;
    e.n = (int) p.n_layers; e.vocab = (int) p.vocab; e.theta = p.theta; e.max_seq = max_seq; e.pf_cap = pf_cap;
    std::vector<lkb_mixer_layer> mdesc(e.n);
    for (int i = 0; i < e.n; ++i) {
        const std::string b = "blk." + std::to_string(i) + ".";
        MixerW m{};
        m.is_attn = p.has(b + "attn_q.qs");
        m.attn_norm = p.f32(b + "attn_norm");
        lkb_mixer_layer d{};
        d.is_attn = m.is_attn; d.attn_norm = m.attn_norm; d.max_seq = max_seq;
        if (m.is_attn) {
            m.wq = q4(p, b + "attn_q"); m.wk = q4(p, b + "attn_k"); m.wv = q4(p, b + "attn_v"); m.out = q4(p, b + "attn_output");
            m.qnorm = p.f32(b + "attn_q_norm"); m.knorm = p.f32(b + "attn_k_norm");
            m.kc = dalloc<uint16_t>((size_t) max_seq * N_KV * HEAD_DIM);       // THE allocation that sizes the context
            m.vc = dalloc<uint16_t>((size_t) max_seq * N_KV * HEAD_DIM);
            d.wq_qs = m.wq.qs; d.wq_d = m.wq.d; d.wk_qs = m.wk.qs; d.wk_d = m.wk.d; d.wv_qs = m.wv.qs; d.wv_d = m.wv.d;
            d.qnorm = m.qnorm; d.knorm = m.knorm; d.kc = m.kc; d.vc = m.vc;
        } else {
            m.in_proj = q4(p, b + "shortconv.in_proj"); m.out = q4(p, b + "shortconv.out_proj");
            m.conv_w = p.f32(b + "shortconv.conv");
            m.hist = dalloc<float>(2 * H);
            d.in_qs = m.in_proj.qs; d.in_d = m.in_proj.d; d.conv_w = m.conv_w; d.hist = m.hist;
        }
        d.out_qs = m.out.qs; d.out_d = m.out.d;
        e.mx.push_back(m); mdesc[i] = d;
        lkb_moe_layer l{};
        l.gate_qs = p.at(b + "ffn_gate_exps.qs"); l.gate_d = p.at(b + "ffn_gate_exps.d");
        l.up_qs = p.at(b + "ffn_up_exps.qs"); l.up_d = p.at(b + "ffn_up_exps.d");
        l.down_qs = p.at(b + "ffn_down_exps.qs"); l.down_d = p.at(b + "ffn_down_exps.d");
        l.router = p.f32(b + "ffn_gate_inp"); l.rbias = p.f32(b + "exp_probs_b"); l.norm_w = p.f32(b + "ffn_norm");
        l.softmax = 0;
        e.moe.push_back(l);
    }
    e.eql = p.at("token_embd.ql"); e.eqh = p.at("token_embd.qh"); e.esc = p.at("token_embd.sc"); e.ed = p.at("token_embd.d");
    e.out_norm = p.f32("output_norm");
    // decode
    e.x = dalloc<float>(H); e.ssq = dalloc<float>(64); e.xq = dalloc<lk::block_q8_1>(64);
    e.logits_v = dalloc<float>(e.vocab);
    const int nb = (e.vocab + 1023) / 1024;
    e.am_v = dalloc<float>(nb); e.am_i = dalloc<int>(nb); e.d_token = dalloc<int>(1); e.d_pos = dalloc<int>(1);
    e.moe_dev = dalloc<lkb_moe_layer>(e.n); e.mixers_dev = dalloc<lkb_mixer_layer>(e.n);
    CK(cudaMemcpy(e.moe_dev, e.moe.data(), e.n * sizeof(lkb_moe_layer), cudaMemcpyHostToDevice));
    CK(cudaMemcpy(e.mixers_dev, mdesc.data(), e.n * sizeof(lkb_mixer_layer), cudaMemcpyHostToDevice));
    e.scratch.logits = dalloc<float>(LKB_MOE_SCRATCH_LOGITS); e.scratch.gu = dalloc<float>(LKB_MOE_SCRATCH_GU);
    e.scratch.sync = dalloc<unsigned>(LKB_MOE_SCRATCH_SYNC);
    e.sscratch.mx = dalloc<float>(LKB_STEP_SCRATCH_MX); e.sscratch.part = dalloc<float>(LKB_STEP_SCRATCH_PART);
    e.np_out = lkb_norm_prod_t{e.out_norm, nullptr, e.xq, e.ssq};
    // prefill
    if (pf_cap > 0) {
        const size_t m = pf_cap, ns = m * TOPK;
        e.max_tiles = (int) (ns / 64) + E;                                      // ref: src/engine.cu:1007
        e.X = dalloc<float>(m * H); e.a_qs = dalloc<int8_t>(m * H); e.a_sc = dalloc<float>(m * BPR * 2); e.inv = dalloc<float>(m);
        e.h32 = dalloc<float>(m * H); e.sel = dalloc<float>(m * E); e.sig = dalloc<float>(m * E);
        e.idx = dalloc<int>(ns); e.w = dalloc<float>(ns); e.cnt = dalloc<int>(E); e.off = dalloc<int>(E);
        e.tiles = dalloc<int>((size_t) e.max_tiles * 4); e.ntiles = dalloc<int>(1); e.perm = dalloc<int>(ns);
        e.a2_qs = dalloc<int8_t>(ns * I); e.a2_sc = dalloc<float>(ns * (I / 32) * 2); e.D = dalloc<float>(ns * H);
        e.Y = dalloc<float>(m * CONV_ROWS); e.o = dalloc<float>(m * H); e.qh = dalloc<uint16_t>(m * H); e.toks = dalloc<int>(m);
        lk::check(lkb_pf_gemm_workspace_bytes(e.max_tiles, H, &e.gemm_ws_bytes), "lkb_pf_gemm_workspace_bytes");
        e.gemm_ws = dalloc<unsigned char>(e.gemm_ws_bytes);
        lk::check(lkb_pf_gemm_set_workspace(e.gemm_ws, e.gemm_ws_bytes), "lkb_pf_gemm_set_workspace");
    }
}

// One decode step: embedding row -> layer 0's norm -> every layer in one persistent launch -> output projection ->
// argmax (stores the next token id and advances the position on the device).  ref: src/engine.cu:480-860
void decode_step(Engine & e, lk::stream_t st) {
    lk::k_embed_q6_K(st, (const uint8_t *) e.eql, (const uint8_t *) e.eqh, (const int8_t *) e.esc, e.ed, e.d_token, H, e.x);
    lk::k_rmsnorm_q8_1(st, e.x, e.mx[0].attn_norm, H, EPS, nullptr, nullptr, e.xq);
    lk::check(lkb_decode_layers(e.moe_dev, e.mixers_dev, e.n, e.x, e.xq, e.d_pos, e.theta, &e.np_out, &e.scratch, &e.sscratch, st),
              "lkb_decode_layers");
    lk::k_gemv_q6_K(st, (const uint8_t *) e.eql, (const uint8_t *) e.eqh, (const int8_t *) e.esc, e.ed, e.xq, e.vocab, SBPR, e.logits_v,
                    e.ssq, EPS);
    lk::k_argmax_part(st, e.logits_v, e.vocab, e.am_v, e.am_i);
    lk::k_argmax_final(st, e.am_v, e.am_i, (e.vocab + 1023) / 1024, e.d_token, e.d_pos);
}

lk::PfGemm gemm_desc(const lk::QT4 * segs, int nseg, const int * seg_end, int N, int bpr, const int8_t * aqs, const float * asc) {
    lk::PfGemm g{};
    for (int i = 0; i < 3; ++i) {
        const int s = i < nseg ? i : nseg - 1;
        g.qs[i] = segs[s].qs; g.d[i] = segs[s].d; g.seg_end[i] = seg_end[i];
    }
    g.N = N; g.bpr = bpr; g.aqs = aqs; g.asc = asc;
    return g;
}

// One chunk of m prompt tokens at positions P .. P+m-1.  ref: src/engine.cu:1024-1250 (pf_chunk)
void prefill_chunk(Engine & e, lk::stream_t st, const int * toks_host, int m, int P) {
    CK(cudaMemcpyAsync(e.toks, toks_host, (size_t) m * 4, cudaMemcpyHostToDevice, (cudaStream_t) st));
    const lk::PfAct a{e.a_qs, e.a_sc}, a2{e.a2_qs, e.a2_sc};
    const int ns = m * TOPK;
    lk::k_pf_embed(st, m, (const uint8_t *) e.eql, (const uint8_t *) e.eqh, (const int8_t *) e.esc, e.ed, e.toks, e.X);
    lk::k_pf_norm(st, m, e.X, e.mx[0].attn_norm, 1, a, e.inv, nullptr);                   // layer 0: a plain norm
    for (int i = 0; i < e.n; ++i) {
        const MixerW & mx = e.mx[i];
        const float * scale = i == 0 ? nullptr : e.inv;
        if (mx.is_attn) {
            const lk::QT4 segs[3] = {mx.wq, mx.wk, mx.wv};
            const int ends[3] = {H, H + N_KV * HEAD_DIM, QKV};
            lk::PfGemm g = gemm_desc(segs, 3, ends, QKV, BPR, e.a_qs, e.a_sc);
            g.ntok = m; g.scale = scale; g.out = e.Y; g.out_ld = QKV;
            lk::pf_gemm_dense(g, st);
            lk::check(lkb_pf_qknr(e.Y, mx.qnorm, mx.knorm, P, e.qh, mx.kc, mx.vc, m, e.theta, st), "k_pf_qknr");
            lk::k_pf_attn(st, e.qh, m, P, mx.kc, mx.vc, e.o);
            lk::k_pf_quant_rows(st, m, e.o, H, BPR, a);
        } else {
            const int ends[3] = {CONV_ROWS, CONV_ROWS, CONV_ROWS};
            lk::PfGemm g = gemm_desc(&mx.in_proj, 1, ends, CONV_ROWS, BPR, e.a_qs, e.a_sc);
            g.ntok = m; g.scale = scale; g.out = e.Y; g.out_ld = CONV_ROWS;
            lk::pf_gemm_dense(g, st);
            lk::k_pf_conv(st, m, e.Y, mx.conv_w, mx.hist, a);
            lk::k_pf_conv_hist(st, e.Y, m, mx.hist);
        }
        {   // out_proj / attn_output, added onto the residual stream
            const int ends[3] = {H, H, H};
            lk::PfGemm g = gemm_desc(&mx.out, 1, ends, H, BPR, e.a_qs, e.a_sc);
            g.ntok = m; g.out = e.X; g.out_ld = H; g.add = 1;
            lk::pf_gemm_dense(g, st);
        }
        // MoE FFN.  ref: src/engine.cu:1170-1241
        const lkb_moe_layer & l = e.moe[i];
        lk::k_pf_norm(st, m, e.X, l.norm_w, 0, a, e.inv, e.h32);
        lk::check(lkb_pf_router_select(e.h32, m, m <= 256, l.router, l.rbias, e.inv, e.sel, e.sig, e.idx, e.w, st), "k_pf_router + k_pf_select");
        lk::check(lkb_zero_i32(e.cnt, E, st), "lkb_zero_i32");
        lk::k_pf_moe_count(st, e.idx, ns, e.cnt);
        lk::k_pf_moe_plan(st, e.cnt, e.off, e.tiles, e.ntiles);
        lk::k_pf_moe_scatter(st, e.idx, ns, e.off, e.perm);
        {
            const lk::QT4 segs[2] = {{l.gate_qs, l.gate_d}, {l.up_qs, l.up_d}};
            const int ends[3] = {I, I, I};
            lk::PfGemm g = gemm_desc(segs, 2, ends, I, BPR, e.a_qs, e.a_sc);
            g.exp_stride = (long long) I * BPR; g.perm = e.perm; g.tiles = e.tiles; g.ntiles = e.ntiles; g.a_shift = 2; g.scale = e.inv;
            g.oqs = e.a2_qs; g.osc = e.a2_sc; g.okb = I / 32;
            lk::pf_gemm_swiglu(g, e.max_tiles, st);
        }
        {
            const lk::QT4 seg{l.down_qs, l.down_d};
            const int ends[3] = {H, H, H};
            lk::PfGemm g = gemm_desc(&seg, 1, ends, H, I / 32, e.a2_qs, e.a2_sc);
            g.exp_stride = (long long) H * (I / 32); g.perm = e.perm; g.tiles = e.tiles; g.ntiles = e.ntiles; g.a_shift = 0;
            g.out = e.D; g.out_ld = H;
            lk::pf_gemm_moe(g, e.max_tiles, st);
        }
        const float * next_norm = i + 1 < e.n ? e.mx[i + 1].attn_norm : e.out_norm;
        lk::k_pf_moe_combine_norm(st, m, e.X, e.D, e.w, next_norm, a, e.inv);
    }
    (void) a2;
}

int env_int(const char * name, int dflt) { const char * v = getenv(name); return v ? atoi(v) : dflt; }

}  // namespace

int main(int argc, char ** argv) {
    setenv("CUDA_MODULE_LOADING", "EAGER", 0);          // module load outside the timed region; an explicit setting wins
    const char * pack = getenv("LK_PACK");
    const char * mode = argc > 1 ? argv[1] : "gen";
    if (!pack) { fprintf(stderr, "LK_PACK not set\n"); return 1; }
    if (strcmp(mode, "gen") != 0) { fprintf(stderr, "unknown mode %s\n", mode); return 1; }
    std::vector<int> toks;
    for (int i = 2; i < argc; ++i) toks.push_back(atoi(argv[i]));
    // a long prompt does not fit an argument list: the same little-endian int32 blob, appended to any argv tokens
    if (const char * pb = getenv("LK_PROMPT_BIN")) {
        FILE * pf = fopen(pb, "rb");
        if (!pf) { fprintf(stderr, "LK_PROMPT_BIN: cannot open %s\n", pb); return 1; }
        if (fseek(pf, 0, SEEK_END) != 0) { fprintf(stderr, "LK_PROMPT_BIN: seek\n"); fclose(pf); return 1; }
        const long nb = ftell(pf);
        rewind(pf);
        if (nb <= 0 || nb % 4 != 0) { fprintf(stderr, "LK_PROMPT_BIN: %s is not a non-empty int32 blob\n", pb); fclose(pf); return 1; }
        const size_t base = toks.size();
        toks.resize(base + (size_t) nb / 4);
        if (fread(toks.data() + base, 4, (size_t) nb / 4, pf) != (size_t) nb / 4) { fprintf(stderr, "LK_PROMPT_BIN: short read\n"); fclose(pf); return 1; }
        fclose(pf);
    }
    if (toks.empty()) { fprintf(stderr, "usage: LK_PACK=<pack> engine gen <token ids ...>   (or LK_PROMPT_BIN=<int32 blob>)\n"); return 1; }
    const int ngen = env_int("LK_NGEN", 32);
    const bool bench = env_int("LK_BENCH", 0) != 0;                      // no per-token output, no stop at end of sequence
    const int eos = env_int("LK_EOS", -1);
    const int pf_chunk = env_int("LK_PF_CHUNK", 4096);
    const int n_prompt = (int) toks.size();
    const int max_seq = env_int("LK_MAX_SEQ", n_prompt + ngen + 8);
    if (ngen < 1 || pf_chunk < 1) { fprintf(stderr, "LK_NGEN and LK_PF_CHUNK must be positive\n"); return 1; }
    if (n_prompt + ngen > max_seq) {
        fprintf(stderr, "prompt (%d) + LK_NGEN (%d) exceeds LK_MAX_SEQ (%d): the KV cache holds LK_MAX_SEQ positions\n", n_prompt, ngen, max_seq);
        return 1;
    }

    CK(cudaSetDevice(env_int("LK_DEVICE", 0)));
    lk::check(lkb_init(env_int("LK_DEVICE", 0)), "lkb_init");
    Engine * e = new Engine();
    e->pk = load_pack(pack);
    for (int t : toks) if (t < 0 || t >= (int) e->pk.vocab) { fprintf(stderr, "token id %d outside the vocabulary (%u)\n", t, e->pk.vocab); return 1; }
    const int nbatch = n_prompt - 1;                                    // all but the last prompt token in chunks
    build(*e, max_seq, nbatch > 0 ? (nbatch < pf_chunk ? nbatch : pf_chunk) : 0);
    cudaStream_t cst;
    CK(cudaStreamCreate(&cst));
    lk::stream_t st = (lk::stream_t) cst;

    // the decode graph, captured once at start-up after one eager step has loaded every kernel
    decode_step(*e, st);
    CK(cudaStreamSynchronize(cst));
    cudaGraph_t graph; cudaGraphExec_t gexec;
    CK(cudaStreamBeginCapture(cst, cudaStreamCaptureModeThreadLocal));
    decode_step(*e, st);
    CK(cudaStreamEndCapture(cst, &graph));
    CK(cudaGraphInstantiate(&gexec, graph, 0));
    // the warm-up step wrote position 0 of the caches, one conv history and advanced the position: start clean
    for (auto & m : e->mx) {
        if (m.is_attn) { CK(cudaMemset(m.kc, 0, (size_t) max_seq * N_KV * HEAD_DIM * 2)); CK(cudaMemset(m.vc, 0, (size_t) max_seq * N_KV * HEAD_DIM * 2)); }
        else CK(cudaMemset(m.hist, 0, 2 * H * sizeof(float)));
    }
    CK(cudaMemset(e->d_pos, 0, 4));
    CK(cudaDeviceSynchronize());

    auto take = [&]() { int t; CK(cudaMemcpy(&t, e->d_token, 4, cudaMemcpyDeviceToHost)); return t; };

    // ---- prompt ----
    auto p0 = std::chrono::steady_clock::now();
    int batches = 0;
    for (int P = 0; P < nbatch; P += pf_chunk, ++batches) prefill_chunk(*e, st, toks.data() + P, (nbatch - P < pf_chunk) ? nbatch - P : pf_chunk, P);
    CK(cudaMemcpyAsync(e->d_pos, &nbatch, 4, cudaMemcpyHostToDevice, cst));
    CK(cudaMemcpyAsync(e->d_token, &toks[nbatch], 4, cudaMemcpyHostToDevice, cst));
    CK(cudaGraphLaunch(gexec, cst));
    CK(cudaStreamSynchronize(cst));
    auto p1 = std::chrono::steady_clock::now();
    const double psec = std::chrono::duration<double>(p1 - p0).count();
    if (lkb_pf_gemm_status() != 0) { fprintf(stderr, "grouped GEMM: a bounded wait expired (status %d)\n", lkb_pf_gemm_status()); return 1; }

    // ---- generation ----
    int next = take(), done = 0;
    bool stopped = false;
    auto t0 = std::chrono::steady_clock::now();
    if (!bench && next == eos) stopped = true;
    else {
        if (!bench) { printf(" %d", next); fflush(stdout); }
        ++done;
        for (int i = 1; i < ngen; ++i) {
            CK(cudaGraphLaunch(gexec, cst));
            CK(cudaStreamSynchronize(cst));
            next = take();
            if (!bench && next == eos) { stopped = true; break; }
            if (!bench) { printf(" %d", next); fflush(stdout); }
            ++done;
        }
    }
    auto t1 = std::chrono::steady_clock::now();
    if (!bench) printf("\n");
    unsigned sync_words[2];
    CK(cudaMemcpy(sync_words, e->scratch.sync, 8, cudaMemcpyDeviceToHost));
    if (sync_words[1] != 0) { fprintf(stderr, "decode step: a bounded wait expired (status %u)\n", sync_words[1]); return 1; }
    const double sec = std::chrono::duration<double>(t1 - t0).count();
    // the first generated token came out of the prompt's last step; the timed loop made done - 1 steps
    const double tps = done > 1 ? (done - 1) / sec : 0.0;
    printf("RESULT ctx=%d generated=%d seconds=%.4f tok_s=%.2f prompt_n=%d prefill_s=%.4f prefill_tok_s=%.2f stopped=%d "
           "prefill_b=%d prefill_batches=%d prefill_mode=%s\n",
           n_prompt + done, done, sec, tps, n_prompt, psec, psec > 0.0 ? n_prompt / psec : 0.0, stopped ? 1 : 0,
           e->pf_cap, batches, nbatch > 0 ? "batch" : "seq");
    return 0;
}
