// Host-side engine: the layer loop of RWKV_x070.forward / forward_batch as kernel launches,
// and the extern "C" surface declared in include/albatross_b200.h.
//
// Two launch programs share the weights:
//   * batch 1, one token (reference/rwkv7.py:128-157): five launches per block —
//       [LN1 + shift-lerps + r/k/v + adapter-down rows] -> [per-head fused WKV] -> [output proj + residual]
//       -> [LN2 + shift-lerp + ffn key + relu^2] -> [ffn value + residual], then [LN_out + head].
//   * any other (B, T) (reference/rwkv7.py:159-221): row-wise LN / lerp kernels, batched matrix
//     products, the same per-head kernel reading precomputed adapter outputs.
#include <stdarg.h>
#include <string.h>

#include <new>
#include <vector>

#include "../../include/albatross_b200.h"
#include "decode.cuh"
#include "gemv_body.cuh"
#include "gemm.cuh"
#include "gemv.cuh"
#include "head.cuh"
#include "rows.cuh"

namespace ab {


static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}
int check_cuda(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return OK;
    set_error("CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
    return ERR_CUDA;
}

static GemvSeg seg_of(const ab_mat& m, const void* mix, int epi, void* out, const void* resid = nullptr) {
    GemvSeg g = {};
    g.w = m.w; g.scale = m.scale; g.col_scale = m.col_scale; g.tscale = m.tscale;
    g.mix = (const __half*)mix; g.resid = (const __half*)resid; g.out = (__half*)out;
    g.fmt = m.fmt; g.epi = epi; g.n_rows = m.n_out; g.K = m.k;
    return g;
}

}  // namespace ab

using namespace ab;

struct ab_model {
    ab_model_desc d;
    std::vector<ab_layer> layers;
    int use_pdl = 1;
    int n_sm = 0;          // blocks of the persistent decode kernel
    int layer_offset = 0;  // pipeline stage: index of this model's first block in the whole network
    int prog_xq_bytes = 0;
    int debug_sync = 0;  // synchronise after every launch and name the one that failed
    int timeline = 0;    // persistent decode kernel records per-phase timestamps
    int timeline_block = 0;   // ... as seen by this block
    // persistent decode kernel, per block: KB of its share of the next matrix-vector phase asked into L2 when it has
    // streamed its last weights of this one, and KB more once the next phase's inputs have arrived (-1: 64 and 128 in
    // dataflow mode, else 0). More than that gets in the way of the blocks that are still streaming.
    int l2_prefetch_kb = -1;
    int l2_prefetch2_kb = -1;
    int smem_prefetch = 0;
    int early_slice = -1;  // first weight slice requested ahead of the input vector: -1 = in dataflow mode only (there it travels
                           // while the block waits for its input anyway; with barriers it delays the input loads and is slower)
    int barrier_prefetch = 0;   // measured slower: the polls of the barrier queue behind the prefetch traffic
    int stage_gemv = 0;  // ab_forward_stage at B = T = 1 runs the batch-1 matrix-vector kernels instead of the row-wise program
    int fuse_heads = 1;  // persistent decode kernel: r/k/v rows of head h on blocks 2h, 2h+1, the adapter down-projections on
                         // the remaining blocks; block 2h runs the head (up-projections from pre-staged weights, WKV step)
                         // as soon as those producers have signalled: two barriers among all blocks fewer per network block
    int pair_split = 16; // ... row groups (of 4 rows) of a head's 48 (r, k, v) that go to block 2h (which also stages the up-projections)
    int merge_ups = 0;   // persistent decode kernel: block h computes the adapter up-projections of head h inside the head
                         // phase: one phase and barrier fewer per block and the same arithmetic as the per-phase
                         // launches (identical logits), but 3 % slower per token than the phase of matrix-vector rows
};

namespace {

inline size_t al(size_t v) { return (v + 255) & ~(size_t)255; }

// Workspace carve-up shared by both programs. M = B*T rows.
struct Workspace {
    __half *x, *xn, *xn2, *r, *k, *v, *vfirst, *att, *kf, *hw, *ha, *hv, *hg;
    __half *mix[6], *w_raw, *a_raw, *vg_raw, *g, *xlast;
    void* gemm_scratch;
    size_t total;
};

int time_mix_down_ops(const ab_layer& L, int layer, const Workspace& ws, GemmOp* ops);
int time_mix_up_ops(const ab_layer& L, int layer, const Workspace& ws, GemmOp* ops);

Workspace carve(const ab_model* m, int B, int T, unsigned char* base) {
    const size_t M = (size_t)B * T, D = m->d.n_embd, F = 4 * D;
    const ab_layer& l0 = m->layers[0];
    size_t rmax[4] = {0, 0, 0, 0};
    for (const ab_layer& l : m->layers) {
        rmax[0] = std::max(rmax[0], (size_t)l.w1t.n_out); rmax[1] = std::max(rmax[1], (size_t)l.a1t.n_out);
        rmax[2] = std::max(rmax[2], (size_t)l.v1t.n_out); rmax[3] = std::max(rmax[3], (size_t)l.g1t.n_out);
    }
    (void)l0;
    Workspace w;
    size_t off = 0;
    auto take = [&](size_t elems) { __half* p = (__half*)(base + off); off += al(elems * 2); return p; };
    // At B = T = 1 the vectors that cross blocks of the persistent kernel may be arrays of tagged 32-bit words
    // (dataflow mode) instead of fp16: twice the room.
    const size_t tw = M == 1 ? 2 : 1;
    w.x = take(tw * M * D); w.xn = take(M * D); w.xn2 = take(M * D);
    w.r = take(tw * M * D); w.k = take(tw * M * D); w.v = take(tw * M * D); w.vfirst = take(M * D); w.att = take(tw * M * D);
    w.kf = take(tw * M * F);
    w.hw = take(tw * M * rmax[0]); w.ha = take(tw * M * rmax[1]); w.hv = take(tw * M * rmax[2]); w.hg = take(tw * M * rmax[3]);
    const bool batched = !(B == 1 && T == 1) || !m->d.emb || !m->d.head.w || m->layer_offset > 0;
    for (int j = 0; j < 6; ++j) w.mix[j] = batched ? take(M * D) : nullptr;
    w.w_raw = take(M * D); w.a_raw = take(M * D); w.vg_raw = take(M * D); w.g = take(M * D);
    w.xlast = batched ? take((size_t)B * D) : nullptr;
    w.gemm_scratch = base + off;
    if (batched) {
        size_t need = m->d.head.w ? gemm_scratch_bytes(m->d.head, (int)M) : 256;
        for (const ab_layer& l : m->layers) {   // the products launched alone may be split along K
            need = std::max(need, gemm_scratch_bytes(l.output, (int)M));
            need = std::max(need, gemm_scratch_bytes(l.ffn_key, (int)M));
            need = std::max(need, gemm_scratch_bytes(l.ffn_value, (int)M));
        }
        for (size_t i = 0; i < m->layers.size(); ++i) {   // the two grouped launches of every block
            GemmOp ops[8];
            int n = time_mix_down_ops(m->layers[i], (int)i + m->layer_offset, w, ops);
            need = std::max(need, gemm_group_scratch_bytes(ops, n, (int)M));
            n = time_mix_up_ops(m->layers[i], (int)i + m->layer_offset, w, ops);
            need = std::max(need, gemm_group_scratch_bytes(ops, n, (int)M));
        }
        off += al(need);
    }
    w.total = off;
    return w;
}

#define AB_TRY(call)                \
    do {                            \
        int _s = (call);            \
        if (_s != OK) return _s;    \
    } while (0)

// Launch + optional post-launch synchronisation that names the failing step.
#define AB_STEP(m, st, layer, what, call)                                                          \
    do {                                                                                           \
        AB_TRY(call);                                                                              \
        if ((m)->debug_sync) {                                                                     \
            cudaError_t _e = cudaStreamSynchronize(st);                                            \
            if (_e != cudaSuccess) {                                                               \
                set_error("layer %d, %s: %s", (layer), (what), cudaGetErrorString(_e));            \
                return ERR_CUDA;                                                                   \
            }                                                                                      \
        }                                                                                          \
    } while (0)

// Pipeline-stage view of a forward pass: where the hidden state comes from and where it goes.
struct StageIO {
    const __half* x_in;   // [M, D] hidden state from the previous stage (null: gather the embedding rows)
    __half* v_first;      // [M, D] layer-0 value, produced by the first stage and read by every later block
    __half* x_out;        // [M, D] hidden state for the next stage (null: final norm + vocabulary head)
};

int forward_one(ab_model* m, const int32_t* token, void* const* state, const Workspace& ws_in, __half* logits,
                cudaStream_t st, const StageIO* io = nullptr) {
    const int D = m->d.n_embd, H = D / HEAD;
    Workspace ws = ws_in;
    if (io && io->v_first) ws.vfirst = io->v_first;
    const bool from_x = io && io->x_in;
    if (from_x) AB_CUDA(cudaMemcpyAsync(ws.x, io->x_in, (size_t)D * 2, cudaMemcpyDeviceToDevice, st));
    const int g0 = m->layer_offset;   // index of this model's first block in the whole network
    for (int i = 0; i < m->d.n_layer; ++i) {
        const ab_layer& L = m->layers[i];
        __half* att_prev = (__half*)state[3 * i];
        float* kv = (float*)state[3 * i + 1];
        __half* ffn_prev = (__half*)state[3 * i + 2];
        {   // LN1 + shift-lerps + r/k/v + adapter-down rows
            GemvParams p = {};
            p.K = D; p.use_pdl = m->use_pdl;
            if (i == 0 && !from_x) { p.emb = (const __half*)m->d.emb; p.token = token; p.emb_rows = m->d.vocab; p.x_copy = ws.x; }
            else p.x = ws.x;
            p.x_prev = att_prev; p.ln_w = (const __half*)L.ln1_w; p.ln_b = (const __half*)L.ln1_b; p.ln_out = ws.xn;
            int n = 0;
            p.seg[n++] = seg_of(L.receptance, L.x_r, EPI_NONE, ws.r);
            p.seg[n++] = seg_of(L.key, L.x_k, EPI_NONE, ws.k);
            p.seg[n++] = seg_of(L.value, L.x_v, EPI_NONE, ws.v);
            p.seg[n++] = seg_of(L.w1t, L.x_w, EPI_TANH, ws.hw);
            p.seg[n++] = seg_of(L.a1t, L.x_a, EPI_NONE, ws.ha);
            if (g0 + i > 0) p.seg[n++] = seg_of(L.v1t, L.x_v, EPI_NONE, ws.hv);
            p.seg[n++] = seg_of(L.g1t, L.x_g, EPI_SIGMOID, ws.hg);
            p.nseg = n;
            AB_STEP(m, st, i, "rkv+adapter-down gemv", gemv_launch(p, st));
        }
        {   // per-head: adapter up-projections, glue, WKV state update, group norm, bonus, gate
            HeadParams h = {};
            h.B = 1; h.T = 1; h.D = D; h.H = H; h.layer0 = (g0 + i == 0);
            h.state = kv; h.r = ws.r; h.k = ws.k; h.v = ws.v; h.v_first = ws.vfirst;
            h.hw = ws.hw; h.ha = ws.ha; h.hv = ws.hv; h.hg = ws.hg;
            h.w2 = (const __half*)L.w2; h.a2 = (const __half*)L.a2; h.v2 = (const __half*)L.v2; h.g2 = (const __half*)L.g2;
            h.rw = L.w1t.n_out; h.ra = L.a1t.n_out; h.rv = (g0 + i == 0) ? 0 : L.v1t.n_out; h.rg = L.g1t.n_out;
            h.w0 = (const __half*)L.w0; h.a0 = (const __half*)L.a0; h.v0 = (const __half*)L.v0;
            h.k_k = (const __half*)L.k_k; h.k_a = (const __half*)L.k_a; h.r_k = (const __half*)L.r_k;
            h.lnx_w = (const __half*)L.lnx_w; h.lnx_b = (const __half*)L.lnx_b;
            h.out = ws.att; h.copy_src = ws.xn; h.copy_dst = att_prev; h.use_pdl = m->use_pdl;
            AB_STEP(m, st, i, "head kernel", head_launch(h, st));
        }
        {   // output projection + residual
            GemvParams p = {};
            p.K = D; p.use_pdl = m->use_pdl; p.x = ws.att; p.nseg = 1;
            p.seg[0] = seg_of(L.output, nullptr, EPI_RESID, ws.x, ws.x);
            AB_STEP(m, st, i, "output gemv", gemv_launch(p, st));
        }
        {   // LN2 + shift-lerp + ffn key + relu^2
            GemvParams p = {};
            p.K = D; p.use_pdl = m->use_pdl; p.x = ws.x; p.nseg = 1;
            p.x_prev = ffn_prev; p.ln_w = (const __half*)L.ln2_w; p.ln_b = (const __half*)L.ln2_b; p.ln_out = ws.xn2;
            p.seg[0] = seg_of(L.ffn_key, L.ffn_x_k, EPI_RELU2, ws.kf);
            AB_STEP(m, st, i, "ffn key gemv", gemv_launch(p, st));
        }
        {   // ffn value + residual; hands the new channel-mix token-shift state over
            GemvParams p = {};
            p.K = 4 * D; p.use_pdl = m->use_pdl; p.x = ws.kf; p.nseg = 1;
            p.seg[0] = seg_of(L.ffn_value, nullptr, EPI_RESID, ws.x, ws.x);
            p.copy_src = ws.xn2; p.copy_dst = ffn_prev; p.copy_n = D;
            AB_STEP(m, st, i, "ffn value gemv", gemv_launch(p, st));
        }
    }
    if (io && io->x_out) {
        AB_CUDA(cudaMemcpyAsync(io->x_out, ws.x, (size_t)D * 2, cudaMemcpyDeviceToDevice, st));
        return OK;
    }
    GemvParams p = {};
    p.K = D; p.use_pdl = m->use_pdl; p.x = ws.x; p.nseg = 1;
    p.ln_w = (const __half*)m->d.lnout_w; p.ln_b = (const __half*)m->d.lnout_b;
    p.seg[0] = seg_of(m->d.head, nullptr, EPI_NONE, logits);
    AB_STEP(m, st, -1, "head gemv", gemv_launch(p, st));
    return OK;
}

// The phase list of one token for the persistent kernel: per block
//   [LN1 + lerps + r/k/v + adapter-down rows] [adapter-up rows] [per-head WKV] [output proj + residual]
//   [LN2 + lerp + ffn key + relu^2] [ffn value + residual], then [LN_out + head].
int build_decode_program(ab_model* m, const int32_t* token, void* const* state, const Workspace& ws, __half* logits,
                         std::vector<unsigned char>& buf, const DecodeProgram* dev_addr) {
    const int D = m->d.n_embd, H = D / HEAD, L = m->d.n_layer;
    const int n_phases = 6 * L + 1;
    const size_t plans_off = decode_plans_offset(n_phases);
    buf.assign(plans_off + sizeof(BlockPlan) * (size_t)n_phases * m->n_sm, 0);
    DecodeProgram* prog = reinterpret_cast<DecodeProgram*>(buf.data());
    prog->n_blocks = m->n_sm;
    prog->plans = reinterpret_cast<const BlockPlan*>((const unsigned char*)dev_addr + plans_off);
    prog->n_phases = n_phases;
    prog->Kn = D;
    prog->xq_bytes = 0;
    prog->first_gemv = 0;
    const bool dataflow_opts = m->fuse_heads && !m->merge_ups;
    prog->l2_prefetch_bytes = (m->l2_prefetch_kb < 0 ? (dataflow_opts ? 64 : 0) : m->l2_prefetch_kb) * 1024;
    prog->l2_prefetch2_bytes = (m->l2_prefetch2_kb < 0 ? (dataflow_opts ? 128 : 0) : m->l2_prefetch2_kb) * 1024;
    // the in-phase adapter up-projection stages its matrices where the prefetched slices would wait: one or the other
    const bool stage_area_taken = m->merge_ups || m->fuse_heads;
    prog->smem_prefetch = stage_area_taken ? 0 : m->smem_prefetch;
    // (dataflow mode: only in the phases that do not stage up-projections into the same area)
    prog->early_slice = m->merge_ups ? 0 : (m->early_slice < 0 ? (m->fuse_heads ? 1 : 0) : m->early_slice);
    prog->barrier_prefetch = stage_area_taken ? 0 : m->barrier_prefetch;
    prog->barrier = const_cast<unsigned*>(&dev_addr->barrier_word);
    prog->epoch = 1;   // tags start above zero: freshly cleared words (tag 0) are "not written yet"
    prog->timeline_block = m->timeline_block;
    prog->timeline_stride = 6u * (unsigned)n_phases;
    prog->timeline = m->timeline ? (unsigned long long*)((unsigned char*)dev_addr +
                                                          decode_timeline_offset(n_phases, m->n_sm)) : nullptr;
    int n = 0;
    // dataflow mode: 1 + index of the phase that wrote the hidden state `ws.x` last (0: plain fp16, barrier mode)
    int x_tag = 0;
    auto gemv_phase = [&](const GemvParams& g) -> int {
        DecodePhase& ph = prog->phases[n++];
        ph.type = PHASE_GEMV;
        ph.g = g;
        AB_TRY(gemv_check(ph.g));
        int xq = 0;
        for (int s = 0; s < ph.g.nseg; ++s) xq += gemv_xq_bytes(ph.g.seg[s].K);
        prog->xq_bytes = std::max(prog->xq_bytes, xq);
        return gemv_check_partials(ph.g, m->n_sm);
    };
    for (int i = 0; i < L; ++i) {
        const ab_layer& Ly = m->layers[i];
        __half* att_prev = (__half*)state[3 * i];
        __half* ffn_prev = (__half*)state[3 * i + 2];
        {
            GemvParams p = {};
            p.K = D;
            if (i == 0) { p.emb = (const __half*)m->d.emb; p.token = token; p.emb_rows = m->d.vocab; p.x_copy = ws.x; }
            else p.x = ws.x;
            p.x_prev = att_prev; p.ln_w = (const __half*)Ly.ln1_w; p.ln_b = (const __half*)Ly.ln1_b; p.ln_out = ws.xn;
            int k = 0;
            p.seg[k++] = seg_of(Ly.receptance, Ly.x_r, EPI_NONE, ws.r);
            p.seg[k++] = seg_of(Ly.key, Ly.x_k, EPI_NONE, ws.k);
            p.seg[k++] = seg_of(Ly.value, Ly.x_v, EPI_NONE, ws.v);
            p.seg[k++] = seg_of(Ly.w1t, Ly.x_w, EPI_TANH, ws.hw);
            p.seg[k++] = seg_of(Ly.a1t, Ly.x_a, EPI_NONE, ws.ha);
            if (i > 0) p.seg[k++] = seg_of(Ly.v1t, Ly.x_v, EPI_NONE, ws.hv);
            p.seg[k++] = seg_of(Ly.g1t, Ly.x_g, EPI_SIGMOID, ws.hg);
            p.nseg = k;
            AB_TRY(gemv_phase(p));
        }
        const int rtot = Ly.w1t.n_out + Ly.a1t.n_out + (i == 0 ? 0 : Ly.v1t.n_out) + Ly.g1t.n_out;
        // dataflow mode ("fuse_heads") needs two blocks per head plus at least four for the adapter rows, whole heads of 16 row groups
        // in the three matrices, and the head's up-projection slices in the idle prefetch area
        const bool fused = m->fuse_heads && !m->merge_ups && 2 * H + 4 <= m->n_sm &&
                           Ly.receptance.n_out == D && Ly.key.n_out == D && Ly.value.n_out == D &&
                           head_ups_smem(rtot) + 8 * 64 * 2 <= (size_t)GEMV_WARPS * GEMV_ROWS * GEMV_SLICE_BYTES &&
                           m->pair_split >= 1 && m->pair_split <= 3 * (HEAD / GEMV_ROWS) - 1;
        AB_CHECK_ARG(i == 0 || fused == (x_tag != 0), "decode program: the blocks of the network must all take the same mode");
        if (fused) {
            DecodePhase& p1 = prog->phases[n - 1];
            p1.no_barrier = 2;         // dataflow: tagged outputs, no barrier among all blocks
            p1.rows_per_block = -1;    // marks the head-aligned plan
            // layer 0 reads the embedding row (weights) and block 0 publishes it as the tagged hidden state
            p1.g.tag_in = i == 0 ? n : x_tag;
            if (i == 0) x_tag = n;
            for (int s = 0; s < p1.g.nseg; ++s) p1.g.seg[s].tag_out = n;
        }
        const bool ups_in_head = fused || (m->merge_ups && H <= m->n_sm && head_ups_smem(rtot) <= gemv_layout(D, 1, 0).total);
        if (!ups_in_head) {   // adapter up-projections: rows of [n_embd, rank], each with its own short input
            GemvParams p = {};
            int k = 0;
            auto up = [&](const ab_mat& mt, const __half* x, __half* out) {
                GemvSeg g = seg_of(mt, nullptr, EPI_NONE, out);
                g.x = x;
                p.seg[k++] = g;
            };
            up(Ly.w2t, ws.hw, ws.w_raw);
            up(Ly.a2t, ws.ha, ws.a_raw);
            if (i > 0) up(Ly.v2t, ws.hv, ws.vg_raw);
            up(Ly.g2t, ws.hg, ws.g);
            p.nseg = k;
            AB_TRY(gemv_phase(p));
        }
        {
            DecodePhase& ph = prog->phases[n++];
            ph.type = PHASE_HEAD;
            HeadParams& h = ph.h;
            h.B = 1; h.T = 1; h.D = D; h.H = H; h.layer0 = (i == 0);
            h.state = (float*)state[3 * i + 1]; h.r = ws.r; h.k = ws.k; h.v = ws.v; h.v_first = ws.vfirst;
            h.w_raw = ws.w_raw; h.a_raw = ws.a_raw; h.vg_raw = ws.vg_raw; h.g = ws.g;
            h.w0 = (const __half*)Ly.w0; h.a0 = (const __half*)Ly.a0; h.v0 = (const __half*)Ly.v0;
            h.k_k = (const __half*)Ly.k_k; h.k_a = (const __half*)Ly.k_a; h.r_k = (const __half*)Ly.r_k;
            h.lnx_w = (const __half*)Ly.lnx_w; h.lnx_b = (const __half*)Ly.lnx_b;
            h.out = ws.att; h.copy_src = ws.xn; h.copy_dst = att_prev;
            if (fused) {
                h.pair_mode = 1; h.tag_in = n - 1; h.tag_out = n;   // n - 1: the phase before (1-based), n: this one
                ph.no_barrier = 2;
            }
            if (ups_in_head) {   // block h computes the adapter outputs of head h itself (no phase, no barrier for them)
                h.hw = ws.hw; h.ha = ws.ha; h.hv = ws.hv; h.hg = ws.hg;
                h.w2 = (const __half*)Ly.w2; h.a2 = (const __half*)Ly.a2; h.v2 = (const __half*)Ly.v2; h.g2 = (const __half*)Ly.g2;
                h.rw = Ly.w1t.n_out; h.ra = Ly.a1t.n_out; h.rv = (i == 0) ? 0 : Ly.v1t.n_out; h.rg = Ly.g1t.n_out;
            }
        }
        {
            GemvParams p = {};
            p.K = D; p.x = ws.att; p.nseg = 1;
            p.seg[0] = seg_of(Ly.output, nullptr, EPI_RESID, ws.x, ws.x);
            if (fused) { p.tag_in = n; p.seg[0].tag_resid = x_tag; p.seg[0].tag_out = n + 1; }   // n: the head phase before
            AB_TRY(gemv_phase(p));
            if (fused) { prog->phases[n - 1].no_barrier = 2; x_tag = n; }
        }
        {
            GemvParams p = {};
            p.K = D; p.x = ws.x; p.nseg = 1;
            p.x_prev = ffn_prev; p.ln_w = (const __half*)Ly.ln2_w; p.ln_b = (const __half*)Ly.ln2_b; p.ln_out = ws.xn2;
            p.seg[0] = seg_of(Ly.ffn_key, Ly.ffn_x_k, EPI_RELU2, ws.kf);
            if (fused) { p.tag_in = x_tag; p.seg[0].tag_out = n + 1; }
            AB_TRY(gemv_phase(p));
            if (fused) prog->phases[n - 1].no_barrier = 2;
        }
        {
            GemvParams p = {};
            p.nseg = 1;
            p.seg[0] = seg_of(Ly.ffn_value, nullptr, EPI_RESID, ws.x, ws.x);
            p.seg[0].x = ws.kf;   // 4*n_embd inputs: read straight from global memory
            p.copy_src = ws.xn2; p.copy_dst = ffn_prev; p.copy_n = D;
            if (fused) { p.seg[0].tag_x = n; p.seg[0].tag_resid = x_tag; p.seg[0].tag_out = n + 1; }   // n: the ffn-key phase before
            AB_TRY(gemv_phase(p));
            if (fused) { prog->phases[n - 1].no_barrier = 2; x_tag = n; }
        }
    }
    GemvParams p = {};
    p.K = D; p.x = ws.x; p.nseg = 1;
    p.ln_w = (const __half*)m->d.lnout_w; p.ln_b = (const __half*)m->d.lnout_b;
    p.seg[0] = seg_of(m->d.head, nullptr, EPI_NONE, logits);
    p.tag_in = x_tag;
    AB_TRY(gemv_phase(p));
    prog->n_phases = n;   // one phase fewer per block when the adapter up-projections run inside the head phase
    int nxt = -1;
    for (int i = n - 1; i >= 0; --i) {
        prog->phases[i].next_gemv = nxt;
        if (prog->phases[i].type == PHASE_GEMV) nxt = i;
    }
    prog->first_gemv = nxt;
    m->prog_xq_bytes = prog->xq_bytes;
    BlockPlan* host_plans = reinterpret_cast<BlockPlan*>(buf.data() + plans_off);
    for (int i = 0; i < n; ++i)
        if (prog->phases[i].type == PHASE_GEMV)
            for (int b = 0; b < m->n_sm; ++b) {
                BlockPlan& bp = host_plans[(size_t)i * m->n_sm + b];
                if (prog->phases[i].rows_per_block > 0) compute_plan_rows(prog->phases[i].g, b, prog->phases[i].rows_per_block, bp);
                else if (prog->phases[i].rows_per_block < 0) compute_plan_heads(prog->phases[i].g, b, m->n_sm, H, m->pair_split, bp);
                else compute_plan(prog->phases[i].g, b, m->n_sm, bp);
            }
    return OK;
}

GemmOp gemm_op(const ab_mat& w, const __half* x, __half* y, int epi, const __half* resid = nullptr) {
    GemmOp o = {};
    o.w = w; o.x = x; o.y = y; o.epi = epi; o.resid = resid;
    return o;
}
int time_mix_down_ops(const ab_layer& L, int layer, const Workspace& ws, GemmOp* ops) {
    int n = 0;
    ops[n++] = gemm_op(L.receptance, ws.mix[0], ws.r, EPI_NONE);
    ops[n++] = gemm_op(L.key, ws.mix[1], ws.k, EPI_NONE);
    ops[n++] = gemm_op(L.value, ws.mix[2], ws.v, EPI_NONE);
    ops[n++] = gemm_op(L.w1t, ws.mix[3], ws.hw, EPI_TANH);
    ops[n++] = gemm_op(L.a1t, ws.mix[4], ws.ha, EPI_NONE);
    ops[n++] = gemm_op(L.g1t, ws.mix[5], ws.hg, EPI_SIGMOID);
    if (layer > 0) ops[n++] = gemm_op(L.v1t, ws.mix[2], ws.hv, EPI_NONE);
    return n;
}
int time_mix_up_ops(const ab_layer& L, int layer, const Workspace& ws, GemmOp* ops) {
    int n = 0;
    ops[n++] = gemm_op(L.w2t, ws.hw, ws.w_raw, EPI_NONE);
    ops[n++] = gemm_op(L.a2t, ws.ha, ws.a_raw, EPI_NONE);
    ops[n++] = gemm_op(L.g2t, ws.hg, ws.g, EPI_NONE);
    if (layer > 0) ops[n++] = gemm_op(L.v2t, ws.hv, ws.vg_raw, EPI_NONE);
    return n;
}

int forward_rows(ab_model* m, int B, int T, const int32_t* tokens, void* const* state, const Workspace& ws_in,
                 __half* logits, int full_output, cudaStream_t st, const StageIO* io = nullptr) {
    const int D = m->d.n_embd, H = D / HEAD, M = B * T;
    Workspace ws = ws_in;
    if (io && io->v_first) ws.vfirst = io->v_first;
    if (io && io->x_in) AB_CUDA(cudaMemcpyAsync(ws.x, io->x_in, (size_t)M * D * 2, cudaMemcpyDeviceToDevice, st));
    else AB_TRY(gather_rows((const __half*)m->d.emb, tokens, M, D, m->d.vocab, ws.x, st));
    const int g0 = m->layer_offset;   // index of this model's first block in the whole network
    for (int li = 0; li < m->d.n_layer; ++li) {
        const int i = li;
        const int gi = g0 + li;
        const ab_layer& L = m->layers[i];
        MixParams mp = {};
        mp.xn = ws.xn; mp.x_prev = (__half*)state[3 * i]; mp.B = B; mp.T = T; mp.D = D; mp.n_mix = 6;
        const void* mv[6] = {L.x_r, L.x_k, L.x_v, L.x_w, L.x_a, L.x_g};
        for (int j = 0; j < 6; ++j) { mp.mix[j] = (const __half*)mv[j]; mp.out[j] = ws.mix[j]; }
        if (ln_mix_rows_ok(mp)) {
            AB_TRY(ln_mix_rows(ws.x, (const __half*)L.ln1_w, (const __half*)L.ln1_b, mp, st, m->use_pdl));
        } else {
            AB_TRY(ln_rows(ws.x, (const __half*)L.ln1_w, (const __half*)L.ln1_b, M, D, 1, 0, ws.xn, st));
            AB_TRY(mix_rows(mp, st));
        }
        void* sc = ws.gemm_scratch;
        {   // r, k, v and the adapter down-projections: one grouped launch
            GemmOp ops[8];
            const int n = time_mix_down_ops(L, gi, ws, ops);
            AB_TRY(gemm_group_launch(ops, n, M, sc, st, m->use_pdl));
        }
        {   // adapter up-projections
            GemmOp ops[8];
            const int n = time_mix_up_ops(L, gi, ws, ops);
            AB_TRY(gemm_group_launch(ops, n, M, sc, st, m->use_pdl));
        }
        HeadParams h = {};
        h.B = B; h.T = T; h.D = D; h.H = H; h.layer0 = (gi == 0);
        h.state = (float*)state[3 * i + 1]; h.r = ws.r; h.k = ws.k; h.v = ws.v; h.v_first = ws.vfirst;
        h.w_raw = ws.w_raw; h.a_raw = ws.a_raw; h.vg_raw = ws.vg_raw; h.g = ws.g;
        h.w0 = (const __half*)L.w0; h.a0 = (const __half*)L.a0; h.v0 = (const __half*)L.v0;
        h.k_k = (const __half*)L.k_k; h.k_a = (const __half*)L.k_a; h.r_k = (const __half*)L.r_k;
        h.lnx_w = (const __half*)L.lnx_w; h.lnx_b = (const __half*)L.lnx_b;
        h.out = ws.att; h.use_pdl = m->use_pdl;
        AB_TRY(head_launch(h, st));
        AB_TRY(gemm_launch(L.output, M, ws.att, ws.x, EPI_RESID, ws.x, sc, st, m->use_pdl));

        MixParams fp = {};
        fp.xn = ws.xn; fp.x_prev = (__half*)state[3 * i + 2]; fp.B = B; fp.T = T; fp.D = D; fp.n_mix = 1;
        fp.mix[0] = (const __half*)L.ffn_x_k; fp.out[0] = ws.mix[0];
        if (ln_mix_rows_ok(fp)) {
            AB_TRY(ln_mix_rows(ws.x, (const __half*)L.ln2_w, (const __half*)L.ln2_b, fp, st, m->use_pdl));
        } else {
            AB_TRY(ln_rows(ws.x, (const __half*)L.ln2_w, (const __half*)L.ln2_b, M, D, 1, 0, ws.xn, st));
            AB_TRY(mix_rows(fp, st));
        }
        AB_TRY(gemm_launch(L.ffn_key, M, ws.mix[0], ws.kf, EPI_RELU2, nullptr, sc, st, m->use_pdl));
        AB_TRY(gemm_launch(L.ffn_value, M, ws.kf, ws.x, EPI_RESID, ws.x, sc, st, m->use_pdl));
    }
    if (io && io->x_out) {
        AB_CUDA(cudaMemcpyAsync(io->x_out, ws.x, (size_t)M * D * 2, cudaMemcpyDeviceToDevice, st));
        return OK;
    }
    if (full_output || T == 1) {
        AB_TRY(ln_rows(ws.x, (const __half*)m->d.lnout_w, (const __half*)m->d.lnout_b, M, D, 1, 0, ws.xn, st));
        return gemm_launch(m->d.head, M, ws.xn, logits, EPI_NONE, nullptr, ws.gemm_scratch, st, m->use_pdl);
    }
    AB_TRY(ln_rows(ws.x, (const __half*)m->d.lnout_w, (const __half*)m->d.lnout_b, B, D, T, T - 1, ws.xlast, st));
    return gemm_launch(m->d.head, B, ws.xlast, logits, EPI_NONE, nullptr, ws.gemm_scratch, st, m->use_pdl);
}

}  // namespace

extern "C" {

const char* ab_last_error(void) { return g_err; }
int ab_version(void) { return 1; }

int ab_device_status(uint32_t* status_host) {
    AB_CHECK_ARG(status_host, "ab_device_status: null pointer");
    AB_CUDA(cudaDeviceSynchronize());
    unsigned int v = 0, zero = 0;
    AB_CUDA(cudaMemcpyFromSymbol(&v, g_device_status, sizeof(v)));
    AB_CUDA(cudaMemcpyToSymbol(g_device_status, &zero, sizeof(zero)));
    *status_host = v;
    if (v != 0) {
        // a wait that gave up may have left split-K arrival counters behind: those of the built-in scratch area are
        // put back to zero here (callers of ab_gemm / ab_forward must clear their own scratch / workspace)
        AB_TRY(static_scratch_reset(nullptr));
        AB_CUDA(cudaDeviceSynchronize());
    }
    return OK;
}

int ab_wkv7_fwd(int B, int T, int C, int H, float* state, const void* r, const void* w, const void* k, const void* v,
                const void* a, const void* b, void* y, void* stream) {
    return wkv7_launch(B, T, C, H, state, (const __half*)r, (const __half*)w, (const __half*)k, (const __half*)v,
                       (const __half*)a, (const __half*)b, (__half*)y, (cudaStream_t)stream);
}

int ab_gemv(const ab_mat* m, const void* x, void* y, void* stream) {
    AB_CHECK_ARG(m && x && y, "ab_gemv: null pointer");
    AB_TRY(check_mat(*m, "ab_gemv"));
    GemvParams p = {};
    p.nseg = 1; p.K = m->k; p.x = (const __half*)x;
    p.use_pdl = 1;   // the kernel reads x and writes y only after its predecessor in the stream has completed
    p.seg[0] = seg_of(*m, nullptr, EPI_NONE, y);
    return gemv_launch(p, (cudaStream_t)stream);
}

size_t ab_gemm_scratch_bytes(const ab_mat* m, int rows) {
    if (!m || rows <= 0 || check_mat(*m, "ab_gemm_scratch_bytes") != OK) return 0;
    return gemm_scratch_bytes(*m, rows);
}

int ab_gemm(const ab_mat* m, int rows, const void* x, void* y, int epi, const void* resid, void* scratch, void* stream) {
    AB_CHECK_ARG(m && x && y, "ab_gemm: null pointer");
    AB_CHECK_ARG(rows > 0, "ab_gemm: rows must be positive");
    AB_TRY(check_mat(*m, "ab_gemm"));
    AB_CHECK_ARG(epi >= EPI_NONE && epi <= EPI_RESID && (epi != EPI_RESID || resid), "ab_gemm: bad epilogue");
    return gemm_launch(*m, rows, (const __half*)x, (__half*)y, epi, (const __half*)resid, scratch, (cudaStream_t)stream);
}

int ab_sample_rows(const void* logits, int rows, int vocab, float noise, uint32_t seed, int32_t* out, void* stream) {
    return sample_rows((const __half*)logits, rows, vocab, noise, seed, out, false, (cudaStream_t)stream);
}

int ab_sample_rows_i64(const void* logits, int rows, int vocab, float noise, uint32_t seed, int64_t* out, void* stream) {
    return sample_rows((const __half*)logits, rows, vocab, noise, seed, out, true, (cudaStream_t)stream);
}

int ab_dequant(const ab_mat* m, float* out, void* stream) {
    AB_CHECK_ARG(m, "ab_dequant: null pointer");
    return dequant_launch(*m, out, (cudaStream_t)stream);
}

int ab_model_create(const ab_model_desc* desc, ab_model** out) {
    AB_CHECK_ARG(desc && out && desc->layers, "ab_model_create: null pointer");
    AB_CHECK_ARG(desc->n_layer > 0 && desc->n_embd > 0 && desc->n_embd % 64 == 0 && desc->vocab > 0,
                 "ab_model_create: bad shape (n_layer=%d n_embd=%d vocab=%d)", desc->n_layer, desc->n_embd, desc->vocab);
    // a pipeline stage may lack the embedding table (not the first stage) or the final norm + head (not the last)
    if (desc->head.w) AB_TRY(check_mat(desc->head, "head.weight"));
    for (int i = 0; i < desc->n_layer; ++i) {
        const ab_layer& l = desc->layers[i];
        const ab_mat* big[6] = {&l.receptance, &l.key, &l.value, &l.output, &l.ffn_key, &l.ffn_value};
        for (const ab_mat* mm : big) AB_TRY(check_mat(*mm, "block matrix"));
        AB_TRY(check_mat(l.w1t, "w1")); AB_TRY(check_mat(l.a1t, "a1")); AB_TRY(check_mat(l.g1t, "g1"));
        if (l.v1t.w) AB_TRY(check_mat(l.v1t, "v1"));
        AB_CHECK_ARG(l.w2 && l.a2 && l.g2, "ab_model_create: layer %d adapter up-projection missing", i);
        AB_CHECK_ARG(l.ln1_w && l.ln1_b && l.ln2_w && l.ln2_b && l.x_r && l.x_w && l.x_k && l.x_v && l.x_a && l.x_g &&
                         l.w0 && l.a0 && l.k_k && l.k_a && l.r_k && l.lnx_w && l.lnx_b && l.ffn_x_k,
                     "ab_model_create: layer %d has a null vector", i);
    }
    ab_model* m = new (std::nothrow) ab_model();
    AB_CHECK_ARG(m, "ab_model_create: out of host memory");
    m->d = *desc;
    m->layers.assign(desc->layers, desc->layers + desc->n_layer);
    m->d.layers = m->layers.data();
    {
        int dev = 0;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&m->n_sm, cudaDevAttrMultiProcessorCount, dev);
        if (m->n_sm <= 0) m->n_sm = 148;
        cudaGetLastError();
    }
    *out = m;
    return OK;
}

void ab_model_destroy(ab_model* m) { delete m; }

size_t ab_workspace_bytes(const ab_model* m, int B, int T) {
    if (!m || B <= 0 || T <= 0) return 0;
    return carve(m, B, T, nullptr).total;
}

size_t ab_decode_program_bytes(const ab_model* m) { return m ? decode_program_bytes(m->d.n_layer, m->n_sm) : 0; }
size_t ab_decode_timeline_offset(const ab_model* m) { return m ? decode_timeline_offset(6 * m->d.n_layer + 1, m->n_sm) : 0; }

int ab_decode_program_build(ab_model* m, const int32_t* token, void* const* state, void* workspace, void* logits,
                            void* program, void* stream) {
    AB_CHECK_ARG(m && token && state && workspace && logits && program, "ab_decode_program_build: null pointer");
    AB_CHECK_ARG(((uintptr_t)workspace & 255) == 0 && ((uintptr_t)program & 255) == 0,
                 "ab_decode_program_build: workspace and program must be 256-byte aligned");
    for (int i = 0; i < 3 * m->d.n_layer; ++i) AB_CHECK_ARG(state[i], "ab_decode_program_build: state[%d] is null", i);
    for (const ab_layer& l : m->layers)
        AB_CHECK_ARG(l.w2t.w && l.a2t.w && l.g2t.w, "ab_decode_program_build: transposed adapter up-projections missing");
    const Workspace ws = carve(m, 1, 1, (unsigned char*)workspace);
    std::vector<unsigned char> buf;
    AB_TRY(build_decode_program(m, token, state, ws, (__half*)logits, buf, (const DecodeProgram*)program));
    // dataflow mode reads "not written yet" from a zero tag: whatever an earlier program or another decode mode left in
    // the workspace must not look like a tagged word
    AB_CUDA(cudaMemsetAsync(workspace, 0, ws.total, (cudaStream_t)stream));
    AB_CUDA(cudaMemcpyAsync(program, buf.data(), buf.size(), cudaMemcpyHostToDevice, (cudaStream_t)stream));
    AB_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    return OK;
}

int ab_decode_run(ab_model* m, void* program, void* stream) {
    AB_CHECK_ARG(m && program, "ab_decode_run: null pointer");
    const DecodeProgram* prog = (const DecodeProgram*)program;
    return decode_launch(prog, const_cast<unsigned*>(&prog->barrier_word), m->d.n_embd, m->prog_xq_bytes, (cudaStream_t)stream);
}

int ab_model_set_option(ab_model* m, const char* name, int value) {
    AB_CHECK_ARG(m && name, "ab_model_set_option: null pointer");
    if (!strcmp(name, "stages")) { (void)value; }   // accepted for compatibility; the streaming depth is fixed
    else if (!strcmp(name, "pdl")) m->use_pdl = value != 0;
    else if (!strcmp(name, "debug_sync")) m->debug_sync = value != 0;
    else if (!strcmp(name, "timeline")) m->timeline = value != 0;
    else if (!strcmp(name, "timeline_block")) m->timeline_block = value < 0 ? -1 : value;
    else if (!strcmp(name, "l2_prefetch_kb")) m->l2_prefetch_kb = value < 0 ? -1 : value;
    else if (!strcmp(name, "l2_prefetch2_kb")) m->l2_prefetch2_kb = value < 0 ? -1 : value;
    else if (!strcmp(name, "smem_prefetch")) m->smem_prefetch = value != 0;
    else if (!strcmp(name, "merge_ups")) m->merge_ups = value != 0;
    else if (!strcmp(name, "fuse_heads")) m->fuse_heads = value != 0;
    else if (!strcmp(name, "pair_split")) m->pair_split = value;
    else if (!strcmp(name, "stage_gemv")) m->stage_gemv = value != 0;
    else if (!strcmp(name, "early_slice")) m->early_slice = value < 0 ? -1 : (value > 2 ? 2 : value);
    else if (!strcmp(name, "barrier_prefetch")) m->barrier_prefetch = value != 0;
    else if (!strcmp(name, "layer_offset")) { AB_CHECK_ARG(value >= 0, "layer_offset must be >= 0"); m->layer_offset = value; }
    else { set_error("unknown option %s", name); return ERR_BAD_ARG; }
    return OK;
}

int ab_forward(ab_model* m, int B, int T, const int32_t* tokens, void* const* state, void* workspace, void* logits,
               int full_output, void* stream) {
    AB_CHECK_ARG(m && tokens && state && workspace && logits, "ab_forward: null pointer");
    AB_CHECK_ARG(B > 0 && T > 0, "ab_forward: bad batch shape B=%d T=%d", B, T);
    AB_CHECK_ARG(((uintptr_t)workspace & 255) == 0, "ab_forward: workspace must be 256-byte aligned");
    for (int i = 0; i < 3 * m->d.n_layer; ++i) AB_CHECK_ARG(state[i], "ab_forward: state[%d] is null", i);
    AB_CHECK_ARG(m->d.emb && m->d.head.w && m->d.lnout_w && m->layer_offset == 0,
                 "ab_forward: this model is a pipeline stage; use ab_forward_stage");
    const Workspace ws = carve(m, B, T, (unsigned char*)workspace);
    if (B == 1 && T == 1) return forward_one(m, tokens, state, ws, (__half*)logits, (cudaStream_t)stream);
    return forward_rows(m, B, T, tokens, state, ws, (__half*)logits, full_output, (cudaStream_t)stream);
}

int ab_forward_stage(ab_model* m, int B, int T, const int32_t* tokens, const void* x_in, void* v_first, void* const* state,
                     void* workspace, void* x_out, void* logits, void* stream) {
    AB_CHECK_ARG(m && state && workspace && v_first, "ab_forward_stage: null pointer");
    AB_CHECK_ARG(B > 0 && T > 0, "ab_forward_stage: bad batch shape B=%d T=%d", B, T);
    AB_CHECK_ARG(((uintptr_t)workspace & 255) == 0, "ab_forward_stage: workspace must be 256-byte aligned");
    AB_CHECK_ARG((x_in != nullptr) != (tokens != nullptr), "ab_forward_stage: give token ids (first stage) or x_in (later stages)");
    AB_CHECK_ARG(!tokens || (m->d.emb && m->layer_offset == 0), "ab_forward_stage: token ids need the embedding table and layer_offset 0");
    AB_CHECK_ARG((x_out != nullptr) != (logits != nullptr), "ab_forward_stage: give x_out (not the last stage) or logits (last stage)");
    AB_CHECK_ARG(!logits || (m->d.head.w && m->d.lnout_w && m->d.lnout_b), "ab_forward_stage: logits need the final norm and head");
    for (int i = 0; i < 3 * m->d.n_layer; ++i) AB_CHECK_ARG(state[i], "ab_forward_stage: state[%d] is null", i);
    const Workspace ws = carve(m, B, T, (unsigned char*)workspace);
    StageIO io = {(const __half*)x_in, (__half*)v_first, (__half*)x_out};
    // stages take the row-wise (batched) program, also at B = T = 1, unless option "stage_gemv" asks for the
    // batch-1 matrix-vector kernels
    if (B == 1 && T == 1 && m->stage_gemv) {
        for (const ab_layer& l : m->layers)
            AB_CHECK_ARG(l.w2 && l.a2 && l.g2, "ab_forward_stage: adapter up-projections missing");
        return forward_one(m, tokens, state, ws, (__half*)logits, (cudaStream_t)stream, &io);
    }
    return forward_rows(m, B, T, tokens, state, ws, (__half*)logits, 0, (cudaStream_t)stream, &io);
}

}  // extern "C"
