#include "executor.h"

#include <algorithm>
#include <cstdint>
#include <stdexcept>
#include <string>

namespace cellm {

namespace {

// ---- signatures of the kernel libraries' entry points (P = pointer, I = int, L = long long, F = float)
typedef void* P;
typedef const void* CP;
typedef int (*EmbedFn)(P out, CP table, int tag, CP ids, int T, int H, int V, float scale, P err, P stream);
typedef int (*AddRmsnormFn)(P x, CP delta, CP w, int w_tag, P y, CP rows, int n, int H, int groups, float eps, int act_tag, P stream);
typedef int (*Add2RmsnormFn)(P x, CP delta, CP delta2, CP w, int w_tag, P y, CP rows, int n, int H, int groups, float eps, int act_tag, P stream);
typedef int (*ResidualAddFn)(P x, CP delta, i64 n, int act_tag, P stream);
typedef int (*SwigluFn)(P h, CP gu, int T, int ff, int tag, int gu_tag, P stream);
typedef int (*ShortConvFn)(P y, CP bcx, CP w, CP bias, int w_tag, P state, i64 slot_stride, CP slot_ids, CP seq, CP cu, int T,
                           int B, int H, int taps, int n_slots, int max_q_len, int act_tag, P err, P stream);
typedef int (*QkNormRopeFn)(P q, CP qkv, i64 row_stride, CP q_w, CP k_w, int w_tag, float eps, CP positions, CP seq, CP bt,
                            int bt_stride, P kp, P vp, int num_pages, int page_size, int T, int nh, int nkv, int hd, int rot,
                            int interleaved, CP inv_freq, int act_tag, P err, P stream);
typedef int (*AttentionPlainFn)(P out, CP q, CP kp, CP vp, CP positions, CP seq, CP bt, int bt_stride, int pages, int page_size,
                                int T, int nh, int nkv, int hd, int hdv, float scale, int window, int tag, P err, P stream);
typedef int (*GemmPlainFn)(P c, CP a, CP w, int M, int N, int K, i64 lda, i64 ldw, i64 ldc, int a_tag, int out_tag, P stream);
typedef int (*AttentionDecodeFn)(P out, P part_o, P part_ml, P counters, CP q, CP kp, CP vp, CP cu, CP ctx, CP bt, int bt_stride,
                                 int B, int T, int pages, int page_size, int nh, int nkv, int hd, float scale, int window,
                                 int nsplit, P err, P stream);
typedef int (*AttentionTcFn)(P out, CP q, CP kp, CP vp, CP cu, CP ctx, CP bt, int bt_stride, int B, int T, int n_tiles, int pages,
                             int page_size, int nh, int nkv, int hd, float scale, int window, P err, P stream);
typedef int (*AttentionFlashFn)(P out, P part_o, P part_ml, CP q, CP kp, CP vp, CP cu, CP ctx, CP bt, int bt_stride, int B, int T,
                                int n_tiles, int pages, int page_size, int nh, int nkv, int hd, float scale, int window, int wide,
                                int nsplit, P err, P stream);
typedef int (*GemmTcFn)(P c, CP a, CP w, int M, int N, int K, i64 lda, i64 ldw, i64 ldc, int out_tag, int bn, int split_k,
                        int epilogue, int w_is_static, P ws, P counters, P err, P stream);
typedef int (*GemmConvFn)(P y, CP a, CP wt, int M, int Nt, int K, i64 lda, i64 ldw, int H, int bn, int split_k, CP taps, CP bias,
                          int ntaps, P state, i64 slot_stride, CP slot_ids, int n_slots, int w_is_static, P err, P stream);
typedef int (*GemmRopeFn)(P q, CP a, CP w, int M, int K, i64 lda, i64 ldw, int bn, int split_k, CP q_w, CP k_w, float eps,
                          CP positions, CP bt, int bt_stride, P kp, P vp, int pages, int page_size, int nh, int nkv, CP inv_freq,
                          int w_is_static, P err, P stream);
typedef int (*GatedNormAddFn)(P x, CP m, CP m_bias, CP gate, i64 gate_ld, int gate_tag, CP gate_bias, CP w, int w_tag, P y, int T, int H, int groups, float eps, int act_tag,
                              P stream);
typedef int (*StreamCastFn)(P y, CP x, i64 n, int act_tag, P stream);
typedef int (*MinGruScanFn)(P out, CP proj, i64 ld, int proj_tag, CP bz, CP bx, int w_tag, P state, i64 slot_stride, CP slot_ids, CP cu,
                            int T, int B, int W, int n_slots, int max_q_len, int act_tag, P err, P stream);
typedef int (*LatentPrepFn)(P q_plain, P q_full, CP proj, i64 ld, int proj_tag, CP c_norm_w, int w_tag, float eps, CP positions, CP seq,
                            CP bt, int bt_stride, P pool, int pages, int page_size, int T, int heads, int dim, int rot_dim, int rank,
                            int rot, int interleaved, CP inv_freq, int act_tag, P err, P stream);
typedef int (*AttentionPlainMaskedFn)(P out, CP q, CP kp, CP vp, CP positions, CP seq, CP bt, int bt_stride, int pages, int page_size,
                                      int T, int nh, int nkv, int hd, int hdv, int v_row, float scale, int window, int keep_first,
                                      CP sinks, float fixed_sink, int has_fixed_sink, CP gate, i64 gate_ld, int tag, P err, P stream);
typedef int (*HeadProductFn)(P out, i64 ldo, i64 out_hs, CP in, i64 ldi, i64 in_hs, CP w, int T, int heads, int N, int K, int tag, P stream);
typedef int (*GatedActFn)(P h, CP gu, i64 ld, CP bg, CP bu, int w_tag, int T, int ff, int act, int tag, int gu_tag, P stream);
typedef int (*BiasAddFn)(P out, CP in, CP b, int w_tag, int T, int N, int tag, P stream);
typedef int (*HeadProductMmaFn)(P out, i64 ldo, i64 out_hs, CP in, i64 ldi, i64 in_hs, CP w, int T, int heads, int N, int K, P stream);
typedef int (*AttentionLatentFn)(P out, P part_o, P part_ml, CP q, CP pool, CP cu, CP ctx, CP bt, int bt_stride, int B, int T, int n_tiles,
                                 int pages, int page_size, int nh, int kw, int dv, float scale, int nsplit, int window, CP sinks, P err,
                                 P stream);
typedef int (*EmbedPosFn)(P out, CP table, int tag, CP ids, CP pos_table, CP positions, int max_pos, int T, int H, int V, float scale, P err,
                          P stream);
typedef int (*AttnPrepFn)(P q, CP qkv, i64 row_stride, CP q_w, CP k_w, int w_tag, float eps, int span, float temp_coef, int temp_every,
                          CP positions, CP seq, CP bt, int bt_stride, P kp, P vp, int num_pages, int page_size, int T, int nh, int nkv,
                          int hd, int hdv, int hq, int hv, int act_tag, P err, P stream);
typedef int (*RouteFn)(P idx, P wts, P gate, CP z, i64 ldz, CP correction, int c_tag, int T, int E, int top, int n_groups, int keep, float scale,
                       int has_gate, P stream);
typedef int (*ExpertsRowwiseFn)(P out, P mid, P smid, CP y, i64 ldy, CP up, CP down, CP sup, CP sdown, CP idx, CP wts, CP gate, int T, int H,
                                int ff, int sff, int top, int E, int act, int tag, P stream);
typedef int (*MoeSortFn)(P row_slot, P slot_row, P tile_group, CP idx, int S, int E, int max_tiles, P stream);
typedef int (*MoeGatherFn)(P xs, CP y, i64 ldy, CP row_slot, CP tile_group, int rows, int top, int H, P stream);
typedef int (*MoeCombineFn)(P out, CP Y, CP slot_row, CP wts, CP shared, CP gate, int T, int H, int top, P stream);
typedef int (*GemmGroupedFn)(P c, CP a, CP w, int M, int N, int K, int groups, i64 lda, i64 ldw, i64 ldc, int out_tag, CP tile_group, int act,
                             P err, P stream);
typedef int (*ActivationFn)(P h, CP u, i64 ld, int T, int n, int act, int tag, P stream);

struct KernelError : std::runtime_error {
    int code;
    KernelError(const char* what, int c) : std::runtime_error(std::string(what) + ": status " + std::to_string(c)), code(c) {}
};

i64 ceil_div(i64 a, i64 b) { return (a + b - 1) / b; }
i64 elt(i64 dtype) { return dtype == EXEC_BF16 ? 2 : 4; }

i64 effective_split(i64 K, i64 split_k) {
    const i64 kblocks = ceil_div(K, 64);
    split_k = std::max<i64>(1, std::min(split_k, kblocks));
    const i64 per = ceil_div(kblocks, split_k);
    return ceil_div(kblocks, per);
}

// Bump allocation out of the step's arena: `x` and the two output slots live for the whole step, the rest of a
// half layer's buffers are given back when the next norm begins.
struct Arena {
    char* base;
    i64 size, top = 0, mark = 0, peak = 0;
    bool dry = false;       // sizes only: nothing is behind the addresses it hands out
    void* take(i64 bytes) {
        const i64 at = (top + 255) & ~(i64)255;
        if (!dry && at + bytes > size) throw std::runtime_error("executor: the step's arena is too small");
        top = at + bytes;
        peak = std::max(peak, top);
        return base + at;
    }
    void keep() { mark = top; }
    void release() { top = mark; }
};

struct Run {
    const ExecProgram& p;
    ExecStep& s;
    Arena arena;
    i64 act;        // element type of the activations
    bool dry = false;       // walk the step and note what it needs, launch nothing
    i64 launches = 0, need_gemm_ws = 0, need_attn_ws = 0;
    // the registers, and the two buffers that native parts leave their outputs in by turns
    ExecRegs regs{};
    void* slot[2] = {nullptr, nullptr};
    int turn = 0;
    // layers whose sublayers read the stream itself: the stream in the activations' type, and whether y holds it now
    void* stream_copy = nullptr;
    bool stream_in_y = false;
    // a bias that the pending result has not taken yet (the gate-and-norm kernel right behind it adds it), and whether
    // the record that runs now may leave its bias so
    const void* pending_bias = nullptr;
    bool may_leave_bias = false;
    // the gate's pre-activations where the sublayer's first product has formed them with its own (rows stacked behind its matrix)
    const void* gate_at = nullptr;
    i64 gate_ld = 0, gate_dtype = 0;

    ExecFn last_fn = FN_COUNT;
    template <typename F> F fn(ExecFn which) {
        if (!p.fns[which]) throw std::runtime_error("executor: entry point " + std::to_string((int)which) + " is not loaded");
        last_fn = which;
        return reinterpret_cast<F>(p.fns[which]);
    }
    void ok(int code, const char* what) {
        if (code != 0) throw KernelError(what, code);
        ++launches;
        if (last_fn < FN_COUNT) ++s.calls[last_fn];
    }
#define LAUNCH(call, what) ok(dry ? 0 : (call), what)

    // ---- products ------------------------------------------------------------------------------------------------
    bool tc_ok(const ExecLinear& l, i64 lda) const { return l.tc_ok && (l.K % 8) == 0 && (lda % 8) == 0; }

    void gemm_plain(void* c, const void* a, const ExecLinear& l, i64 M, i64 N, i64 lda, i64 out_dtype) {
        LAUNCH(fn<GemmPlainFn>(FN_GEMM_PLAIN)(c, a, l.w, (int)M, (int)N, (int)l.K, lda, l.ldw, N, (int)act, (int)out_dtype, s.stream),
           "gemm_plain");
    }

    // The tensor-core product with a given tile shape and split; c: [M, N] (or [M, N/2] with the SwiGLU epilogue).
    void gemm_tc(void* c, const void* a, const ExecLinear& l, i64 M, i64 N, i64 lda, i64 out_dtype, i64 bn, i64 split_k,
                 i64 epilogue, i64 ldc = -1) {
        if (ldc < 0) ldc = epilogue ? N / 2 : N;
        const i64 split = effective_split(l.K, split_k);
        // swapped tiles whose K split is one thread-block cluster (2..8 CTAs) sum their pieces through shared
        // memory: no workspace, no counters
        const bool in_cluster = bn < 0 && ((split >= 2 && split <= 8) || (split == 1 && epilogue == 1));
        const bool through_ws = !in_cluster && (split > 1 || (epilogue == 1 && bn < 0));
        void* ws = nullptr;
        if (through_ws) {
            need_gemm_ws = std::max(need_gemm_ws, split * M * N);
            if (!dry && split * M * N > s.gemm_ws_floats) throw std::runtime_error("executor: the products' workspace is too small");
            ws = s.gemm_ws;
        }
        // plain tiles leave the sum of their K-split pieces to a second kernel; swapped tiles outside a cluster let
        // the last CTA of a tile sum them
        void* counters = (split > 1 && !in_cluster && bn < 0) ? s.counters : nullptr;
        LAUNCH(fn<GemmTcFn>(FN_GEMM_TCGEN05)(c, a, l.w, (int)M, (int)N, (int)l.K, lda, l.ldw, ldc, (int)out_dtype, (int)bn,
                                         (int)split_k, (int)epilogue, (int)p.static_flag, ws, counters, s.err, s.stream),
           "gemm_tcgen05");
        if (bn > 0 && split > 1) ++launches;          // the kernel that sums the K-split pieces
    }

    // a [M, K] (row pitch lda) . w^T -> c [M, N] of out_dtype
    void product(void* c, const void* a, const ExecLinear& l, i64 M, i64 lda, i64 out_dtype, i64 N = -1) {
        if (N < 0) N = l.N;
        if (l.dtype != act) throw std::runtime_error("executor: a weight whose element type differs from the activations'");
        if (act == EXEC_F32 || !tc_ok(l, lda)) {
            gemm_plain(c, a, l, M, N, lda, out_dtype);
        } else {
            i64 bn, split;
            plan_tiles(M, N, l.K, p.sms, &bn, &split);
            gemm_tc(c, a, l, M, N, lda, out_dtype, bn, split, 0);
        }
    }
    // out[t, h * out_hs + n] = sum_k in[t, h * in_hs + k] * w[h][n][k] for per-head matrices w [heads, N, K]: many tokens
    // under bfloat16 run on the tensor cores, all heads in one launch where K fits two tiles in shared memory (else the
    // tcgen05 product once a head); the rest one plain kernel over all heads
    void head_products(void* out, i64 ldo, i64 out_hs, const void* in, i64 ldi, i64 in_hs, const void* w, i64 T, i64 heads, i64 N,
                       i64 K) {
        const bool tc = act == EXEC_BF16 && T > 16 && K % 8 == 0 && ldi % 8 == 0 && in_hs % 8 == 0 && (N * K) % 8 == 0 &&
                        ((uintptr_t)in % 16) == 0 && ((uintptr_t)w % 16) == 0;
        if (tc && K % 16 == 0 && K <= 512) {
            LAUNCH(fn<HeadProductMmaFn>(FN_HEAD_PRODUCT_MMA)(out, ldo, out_hs, in, ldi, in_hs, w, (int)T, (int)heads, (int)N, (int)K, s.stream),
                   "head_product_mma");
            return;
        }
        if (!tc || T < 128) {
            LAUNCH(fn<HeadProductFn>(FN_HEAD_PRODUCT)(out, ldo, out_hs, in, ldi, in_hs, w, (int)T, (int)heads, (int)N, (int)K, (int)act,
                                                  s.stream),
                   "head_product");
            return;
        }
        i64 bn, split;
        plan_tiles(T, N, K, p.sms, &bn, &split);
        for (i64 h = 0; h < heads; ++h) {
            ExecLinear l{static_cast<const char*>(w) + h * N * K * 2, N, K, K, EXEC_BF16, 1};
            gemm_tc(static_cast<char*>(out) + h * out_hs * 2, static_cast<const char*>(in) + h * in_hs * 2, l, T, N, ldi, act, bn, split,
                    0, ldo);
        }
    }
    void* linear(const void* a, const ExecLinear& l, i64 M, i64 lda, i64 out_dtype, i64 N = -1) {
        void* c = arena.take(M * (N < 0 ? l.N : N) * elt(out_dtype));
        product(c, a, l, M, lda, out_dtype, N);
        return c;
    }

    // the plan of a decode product with an epilogue of its own, or false
    bool epilogue_plan(i64 M, i64 N, i64 K, i64* bn, i64* split) const {
        plan_tiles(M, N, K, p.sms, bn, split);
        return *bn < 0 && ceil_div(M, -*bn) == 1 && effective_split(K, *split) <= 8;
    }

    // ---- registers -----------------------------------------------------------------------------------------------
    // A part's output becomes an addend that waits for the next norm. Two may wait at once (a layer whose mixer and
    // feed-forward read the same norm's output): regs.pending, the older, and pending2. They lie in the two output
    // slots, so before a third part writes, the older one goes into the stream.
    const void* pending2 = nullptr;
    void add_older_now() {
        if (!regs.pending) return;
        LAUNCH(fn<ResidualAddFn>(FN_RESIDUAL_ADD)(regs.x, regs.pending, s.T * p.H, (int)act, s.stream), "residual_add");
        stream_in_y = false;
        regs.pending = pending2;
        pending2 = nullptr;
    }
    // for what knows one addend only (a Python part, the stream's readers): the second joins the stream at once
    void one_addend() {
        if (!pending2) return;
        LAUNCH(fn<ResidualAddFn>(FN_RESIDUAL_ADD)(regs.x, pending2, s.T * p.H, (int)act, s.stream), "residual_add");
        stream_in_y = false;
        pending2 = nullptr;
    }
    void set_pending(const void* out) {
        if (!regs.pending) regs.pending = out;
        else if (!pending2) pending2 = out;
        else throw std::runtime_error("executor: three addends wait");
    }
    const void* input() const {
        if (!regs.y) throw std::runtime_error("executor: a part wants activations before any norm has left some");
        return regs.y;
    }

    void embed(const EmbedParams& e) {
        if (e.pos_table)
            LAUNCH(fn<EmbedPosFn>(FN_EMBED_POS)(regs.x, e.table, (int)e.dtype, s.ids, e.pos_table, s.positions, (int)e.max_pos, (int)s.T, (int)p.H,
                                            (int)p.V, (float)e.scale, s.err, s.stream),
               "embed_pos");
        else
        LAUNCH(fn<EmbedFn>(FN_EMBED)(regs.x, e.table, (int)e.dtype, s.ids, (int)s.T, (int)p.H, (int)p.V, (float)e.scale, s.err, s.stream),
           "embed");
        stream_in_y = false;
    }
    void rms_norm(const RmsNormParams& n) {
        const bool rows = regs.phase == 2;
        arena.release();
        const i64 count = rows ? s.R : s.T;
        void* y = arena.take(count * p.H * elt(act));
        if (pending2)
            LAUNCH(fn<Add2RmsnormFn>(FN_ADD2_RMSNORM)(regs.x, regs.pending, pending2, n.w, (int)n.dtype, y, rows ? s.rows : nullptr, (int)count,
                                                  (int)p.H, (int)std::max<i64>(n.groups, 1), (float)n.eps, (int)act, s.stream),
                   "add2_rmsnorm");
        else
        LAUNCH(fn<AddRmsnormFn>(FN_ADD_RMSNORM)(regs.x, regs.pending, n.w, (int)n.dtype, y, rows ? s.rows : nullptr, (int)count, (int)p.H,
                                            (int)std::max<i64>(n.groups, 1), (float)n.eps, (int)act, s.stream),
           "add_rmsnorm");
        if (!rows) regs.pending = pending2 = nullptr;      // with rows given the stream itself is not touched
        regs.y = y;
        stream_in_y = false;
    }
    void head(const HeadParams& h) {
        if (regs.phase != 2) throw std::runtime_error("executor: the output product belongs to the epilogue");
        if (h.w.dtype != act) throw std::runtime_error("executor: a head whose element type differs from the activations'");
        product(regs.logits, input(), h.w, s.R, p.H, EXEC_F32);
    }
    void python(const PythonParams& py) {
        if (dry) {
            // the sizing walk calls no Python part: a native part behind one (a head behind a Python norm) finds an
            // address that stands for the activations the part will leave (never read in this walk)
            if (!regs.y) regs.y = arena.base;
            return;
        }
        if (!p.python) throw std::runtime_error("executor: a Python part in a program without a callback");
        one_addend();
        stream_in_y = false;
        if (p.python(py.token, &regs) != 0) throw std::runtime_error("executor: a Python part raised");
    }

    // y = the stream in the activations' type (the 32-bit stream itself when the activations are 32-bit)
    void read_stream() {
        one_addend();
        if (stream_in_y) return;
        if (regs.pending) {
            LAUNCH(fn<ResidualAddFn>(FN_RESIDUAL_ADD)(regs.x, regs.pending, s.T * p.H, (int)act, s.stream), "residual_add");
            regs.pending = nullptr;
        }
        arena.release();
        if (act == EXEC_F32) {
            regs.y = regs.x;
        } else {
            if (!stream_copy) {
                stream_copy = arena.take(s.T * p.H * elt(act));
                arena.keep();
            }
            LAUNCH(fn<StreamCastFn>(FN_STREAM_CAST)(stream_copy, regs.x, s.T * p.H, (int)act, s.stream), "stream_cast");
            regs.y = stream_copy;
        }
        stream_in_y = true;
    }
    // the waiting result of a sublayer, gated by a product over the sublayer's input (still in y), normed in groups
    // and added into the stream; y = the new stream
    void gated_norm_add(const GatedNormAddParams& n) {
        if (!regs.pending) throw std::runtime_error("executor: a gate and norm without a sublayer's result before them");
        if (regs.phase != 1) throw std::runtime_error("executor: a gate and norm outside the layers");
        if (pending2) throw std::runtime_error("executor: a gate and norm with two results before them");
        const i64 T = s.T, H = p.H;
        const void* g = nullptr;
        i64 g_ld = H, g_dtype = act;
        if (n.stacked) {
            if (!gate_at) throw std::runtime_error("executor: a stacked gate whose sublayer left no gate");
            g = gate_at, g_ld = gate_ld, g_dtype = gate_dtype;
        } else if (n.gate.w) {
            g = linear(input(), n.gate, T, H, act);
        }
        gate_at = nullptr;
        // without a copy of the stream yet (no sublayer of this pass has read the stream so far) y is left to the next reader
        void* y = act != EXEC_F32 ? stream_copy : nullptr;
        const void* m_bias = pending_bias;
        pending_bias = nullptr;
        LAUNCH(fn<GatedNormAddFn>(FN_GATED_NORM_ADD)(regs.x, regs.pending, m_bias, g, g_ld, (int)g_dtype, n.gate_bias, n.w, (int)n.w_dtype, y, (int)T, (int)H,
                                                 (int)std::max<i64>(n.groups, 1), (float)n.eps, (int)act, s.stream),
           "gated_norm_add");
        regs.pending = nullptr;
        regs.y = act == EXEC_F32 ? regs.x : y;
        stream_in_y = regs.y != nullptr;
        arena.release();
    }

    void feed_forward(const SwiGLUParams& L, const void* x, void* out);
    void gated_mlp(const GatedMlpParams& L, const void* x, void* out);
    void routed_mlp(const RoutedMlpParams& L, const void* x, void* out);
    void mingru(const MinGruParams& L, const ExecItem& it, const void* x, void* out);
    void latent_attention(const LatentAttentionParams& L, const ExecItem& it, const void* x, void* out);
    void short_conv(const ShortConvParams& L, const ExecItem& it, const void* x, void* out);
    void attention(const AttentionParams& L, const ExecItem& it, const void* x, void* out);
    void* attend(const AttentionParams& L, const ExecItem& it, const void* q, void* o = nullptr);

    // a mixer or feed-forward record: reads `in`, writes `out`
    void produce(const ExecOp& op, const ExecItem* it, const void* in, void* out) {
        switch (op.kind) {
            case OP_SHORT_CONV:
                if (!it) throw std::runtime_error("executor: a mixer outside the layers");
                short_conv(*static_cast<const ShortConvParams*>(op.params), *it, in, out);
                break;
            case OP_ATTENTION:
                if (!it) throw std::runtime_error("executor: a mixer outside the layers");
                attention(*static_cast<const AttentionParams*>(op.params), *it, in, out);
                break;
            case OP_SWIGLU: feed_forward(*static_cast<const SwiGLUParams*>(op.params), in, out); break;
            case OP_GATED_MLP: gated_mlp(*static_cast<const GatedMlpParams*>(op.params), in, out); break;
            case OP_ROUTED_MLP: routed_mlp(*static_cast<const RoutedMlpParams*>(op.params), in, out); break;
            case OP_MINGRU:
                if (!it) throw std::runtime_error("executor: a mixer outside the layers");
                mingru(*static_cast<const MinGruParams*>(op.params), *it, in, out);
                break;
            case OP_LATENT_ATTENTION:
                if (!it) throw std::runtime_error("executor: a mixer outside the layers");
                latent_attention(*static_cast<const LatentAttentionParams*>(op.params), *it, in, out);
                break;
            case OP_LINEAR: {
                const LinearParams& l = *static_cast<const LinearParams*>(op.params);
                product(out, in, l.w, s.T, l.lda, l.out_dtype);
                break;
            }
            case OP_ATTEND: {
                if (!it) throw std::runtime_error("executor: attention outside the layers");
                attend(*static_cast<const AttentionParams*>(op.params), *it, in, out);
                break;
            }
            default: throw std::runtime_error("executor: record kind " + std::to_string(op.kind) + " produces nothing");
        }
    }

    void run(const ExecOp& op) {
        const ExecItem* it = regs.phase == 1 ? &s.items[regs.item] : nullptr;
        switch (op.kind) {
            case OP_EMBED: embed(*static_cast<const EmbedParams*>(op.params)); break;
            case OP_RMS_NORM: rms_norm(*static_cast<const RmsNormParams*>(op.params)); break;
            case OP_HEAD: head(*static_cast<const HeadParams*>(op.params)); break;
            case OP_PYTHON: python(*static_cast<const PythonParams*>(op.params)); break;
            case OP_READ_STREAM: read_stream(); break;
            case OP_GATED_NORM_ADD: gated_norm_add(*static_cast<const GatedNormAddParams*>(op.params)); break;
            case OP_SHORT_CONV: case OP_ATTENTION: case OP_SWIGLU: case OP_MINGRU: case OP_LATENT_ATTENTION: case OP_GATED_MLP: case OP_ROUTED_MLP: {
                if (regs.pending && pending2) add_older_now();      // both output slots are taken: the older addend's is written next
                void* out = slot[turn];
                produce(op, it, input(), out);
                set_pending(out);
                turn ^= 1;
                break;
            }
            default: throw std::runtime_error("executor: unknown record kind " + std::to_string(op.kind));
        }
    }
    void run(const ExecOps& ops) {
        for (i64 i = 0; i < ops.n; ++i) {
            // a feed-forward whose result goes straight into a gate-and-norm kernel leaves its last bias to that kernel
            may_leave_bias = false;
            if (ops.ops[i].kind == OP_GATED_MLP && i + 1 < ops.n && ops.ops[i + 1].kind == OP_GATED_NORM_ADD) {
                const GatedMlpParams& f = *static_cast<const GatedMlpParams*>(ops.ops[i].params);
                const GatedNormAddParams& n = *static_cast<const GatedNormAddParams*>(ops.ops[i + 1].params);
                may_leave_bias = f.b_dtype == n.w_dtype;
            }
            run(ops.ops[i]);
        }
        may_leave_bias = false;
    }
};

}  // namespace

void plan_tiles(i64 M, i64 N, i64 K, i64 sms, i64* bn_out, i64* split_out) {
    const i64 kblocks = ceil_div(K, 64);
    if (M <= 64) {
        // Swapped tiles: 128 weight rows by 16, 32 or 64 tokens. Enough CTAs to fill the SMs, and no CTA with much
        // more than ~300 KB of weights to stream by itself; at most 8 (the split of a tile is one thread-block
        // cluster) and at least four K blocks each. Products with tiles to spare are not split.
        const i64 narrow = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
        const i64 tiles = ceil_div(N, 128);
        i64 split;
        if (tiles >= 2 * sms) {
            split = 1;
        } else {
            const i64 fill = ceil_div(sms * 85 / 100, tiles);
            const i64 stream = ceil_div(128 * K * 2, 300 * 1024);
            split = std::max<i64>(1, std::min({std::max(fill, stream), kblocks / 4, (i64)8}));
        }
        *bn_out = -narrow;
        *split_out = split;
        return;
    }
    i64 bn = N >= 256 ? 256 : (N > 64 ? 128 : 64);
    if (bn == 256 && kblocks >= 64 && M > 256 && ceil_div(N, 256) * ceil_div(M, 128) < sms / 2) {
        // A long K (the feed-forward's way back), three row tiles or more, too few tiles of 128 x 256 for the SMs: those tiles stay, whose
        // products run nearer the tensor pipe's rate than narrower ones, and K is split until the SMs are filled; the
        // pieces go through the workspace and a second kernel sums them.
        const i64 t256 = ceil_div(N, 256) * ceil_div(M, 128);
        *bn_out = 256;
        *split_out = std::max<i64>(1, std::min({ceil_div(sms * 85 / 100, t256), kblocks / 4, (i64)16}));
        return;
    }
    if (bn == 256) {
        // The persistent kernel takes any width from 128 to 256 in steps of 16. A tile costs about 0.1 + 0.9 * width / 256
        // of a 256-wide one (a 128-wide one 0.55); the width whose waves finish soonest wins, the wider on a tie: it
        // is the one whose number of tiles comes closest to a multiple of the SMs from below.
        const i64 mt = ceil_div(M, 128);
        double best = 1e30;
        for (i64 w = 256; w >= 128; w -= 16) {
            const double cost = (double)ceil_div(mt * ceil_div(N, w), sms) * (0.1 + 0.9 * (double)w / 256.0);
            if (cost < best * 0.98) { best = cost; bn = w; }
        }
    }
    i64 tiles = ceil_div(N, bn) * ceil_div(M, 128);
    if (tiles < sms / 2) {
        // Too few plain tiles to fill the GPU (a few hundred tokens, or a narrow product).
        if (M <= 128) {
            // up to two token tiles: swapped tiles of 128 weight rows by 64 tokens, the K split summed in a cluster
            // (as for fewer tokens, no CTA with much more than ~300 KB of weights to stream by itself)
            const i64 stiles = ceil_div(N, 128) * ceil_div(M, 64);
            const i64 want = sms * 85 / 100;
            const i64 stream = ceil_div(128 * K * 2, 300 * 1024);
            *bn_out = -64;
            *split_out = stiles >= want ? 1 : std::max<i64>(1, std::min({std::max(ceil_div(want, stiles), stream), kblocks / 4, (i64)8}));
            return;
        }
        // more tokens: tiles of 128 x 128 with K split until the SMs are filled; the pieces go through the
        // workspace and a second kernel sums them
        bn = N > 64 ? 128 : 64;
        tiles = ceil_div(N, bn) * ceil_div(M, 128);
        *bn_out = bn;
        *split_out = std::max<i64>(1, std::min({ceil_div(sms * 85 / 100, tiles), kblocks / 4, (i64)16}));
        return;
    }
    *bn_out = bn;
    *split_out = 1;
}

namespace {

void Run::feed_forward(const SwiGLUParams& L, const void* x, void* out) {
    const i64 T = s.T, H = p.H;
    void* h;
    if (L.fused && act == EXEC_BF16 && tc_ok(L.gate_up, H)) {
        i64 bn, split;
        plan_tiles(T, L.gate_up.N, L.gate_up.K, p.sms, &bn, &split);
        if (bn == 64) bn = 128;
        else if (bn > 128 && bn < 256) bn = 256;       // gate and up blocks of 64: widths of 128 and 256 only
        h = arena.take(T * L.ff * elt(act));
        gemm_tc(h, x, L.gate_up, T, L.gate_up.N, H, act, bn, split, 1);
    } else if (L.fused) {
        throw std::runtime_error("executor: activations do not fit the fused SwiGLU kernel");
    } else {
        // gate and up stay in 32-bit until silu(g) * u is formed, as in the fused epilogue: one rounding, not three
        void* gu = linear(x, L.gate_up, T, H, EXEC_F32);
        h = arena.take(T * L.ff * elt(act));
        LAUNCH(fn<SwigluFn>(FN_SWIGLU)(h, gu, (int)T, (int)L.ff, (int)act, (int)EXEC_F32, s.stream), "swiglu");
    }
    product(out, h, L.down, T, L.ff, act);
}

void Run::short_conv(const ShortConvParams& L, const ExecItem& it, const void* x, void* out) {
    const i64 T = s.T, H = p.H;
    void* y = nullptr;
    if (p.fused_conv && L.in_proj_tiled && s.max_q_len == 1 && act == EXEC_BF16) {
        ExecLinear tiled = L.in_proj;
        tiled.w = L.in_proj_tiled;
        tiled.N = L.tiled_rows;
        tiled.ldw = L.in_proj.K;
        i64 bn, split;
        if (tc_ok(tiled, H) && epilogue_plan(T, L.tiled_rows, H, &bn, &split)) {
            y = arena.take(T * H * elt(act));
            LAUNCH(fn<GemmConvFn>(FN_GEMM_CONV)(y, x, L.in_proj_tiled, (int)T, (int)L.tiled_rows, (int)H, H, tiled.ldw, (int)H, (int)bn,
                                            (int)split, L.taps, L.bias, (int)L.n_taps, it.state, it.slot_stride, s.slot_ids,
                                            (int)it.n_slots, (int)p.static_flag, s.err, s.stream),
               "gemm_conv_tcgen05");
        }
    }
    if (!y) {
        void* bcx = linear(x, L.in_proj, T, H, act);
        y = arena.take(T * H * elt(act));
        LAUNCH(fn<ShortConvFn>(FN_SHORT_CONV)(y, bcx, L.taps, L.bias, (int)L.taps_dtype, it.state, it.slot_stride, s.slot_ids,
                                          s.seq_of_token, s.cu_seqlens, (int)T, (int)s.B, (int)H, (int)L.n_taps, (int)it.n_slots,
                                          (int)s.max_q_len, (int)act, s.err, s.stream),
           "short_conv");
        if (L.n_taps > 1 && !(s.max_q_len > 0 && s.max_q_len <= 4)) ++launches;     // the state update is a launch of its own
    }
    product(out, y, L.out_proj, T, H, act);
}

void* Run::attend(const AttentionParams& L, const ExecItem& it, const void* q, void* o) {
    const i64 T = s.T, nh = L.nh, nkv = L.nkv, hd = L.hd, hdv = L.hdv > 0 ? L.hdv : L.hd;
    if (!o) o = arena.take(T * nh * hdv * elt(act));
    const float scale = (float)L.scale;
    if (act == EXEC_BF16 && (hd == 32 || hd == 64 || hd == 128) && hdv == hd && L.scale > 0) {
        const i64 G = nh / nkv;
        if (s.max_q_len * G <= 16) {
            // decoded tokens: one CTA per (request, kv head, piece of the keys)
            const i64 blocks = ceil_div(s.max_total_len, 64);
            // Pieces of the keys: as many as fill four CTAs an SM, of four blocks of 64 keys or more. Where that asks for
            // more than one cluster of eight, pieces of two blocks and a multiple of eight of them: clusters of eight
            // combine their pieces in shared memory and only one piece a cluster goes through the workspace.
            const i64 fill = 4 * p.sms / (s.B * nkv);
            i64 nsplit = std::max<i64>(1, std::min(fill, blocks / 4));
            if (blocks / 4 > 8) nsplit = std::max<i64>(1, std::min(fill, blocks / 2));
            if (nsplit >= 16) nsplit = nsplit / 8 * 8;
            void *part_o = nullptr, *part_ml = nullptr, *counters = nullptr;
            if (nsplit > 8) {          // up to 8 pieces meet inside a thread-block cluster and need no workspace
                if (s.B * nkv > p.max_counters) throw std::runtime_error("executor: too many (request, kv head) pairs for the counters");
                const i64 rows = T * nh;
                need_attn_ws = std::max(need_attn_ws, nsplit * rows * (hd + 2));
                if (!dry && nsplit * rows * (hd + 2) > s.attn_ws_floats) throw std::runtime_error("executor: the attention workspace is too small");
                part_o = s.attn_ws;
                part_ml = (float*)s.attn_ws + nsplit * rows * hd;
                counters = s.counters;
            }
            LAUNCH(fn<AttentionDecodeFn>(FN_ATTENTION_DECODE)(o, part_o, part_ml, counters, q, it.k, it.v, s.cu_seqlens, s.ctx_lens,
                                                          it.block_table, (int)it.bt_stride, (int)s.B, (int)T, (int)it.num_pages,
                                                          (int)it.page_size, (int)nh, (int)nkv, (int)hd, scale, (int)L.window,
                                                          (int)nsplit, s.err, s.stream),
               "attention_decode");
            return o;
        }
        // prompt portions that fill the tcgen05 kernel's pairs of 128-row tiles and enough CTAs (below that the
        // mma.sync kernel with its split over the keys fills the GPU better)
        const i64 ps = it.page_size;
        if (hd == 64 && G <= 128 && 128 % G == 0 && (ps == 8 || ps == 16 || ps == 32 || ps == 64 || ps == 128)) {
            const i64 per_tile = 256 / G;
            i64 tc_tiles = 0;
            for (i64 b = 0; b < s.B; ++b) tc_tiles += ceil_div(s.q_lens[b], per_tile);
            const i64 min_ctas = p.tc_min_ctas < 0 ? p.sms / 8 : p.tc_min_ctas;
            if (tc_tiles * nkv >= min_ctas && (double)T >= p.tc_min_fill * (double)(tc_tiles * per_tile)) {
                LAUNCH(fn<AttentionTcFn>(FN_ATTENTION_TC)(o, q, it.k, it.v, s.cu_seqlens, s.ctx_lens, it.block_table, (int)it.bt_stride,
                                                      (int)s.B, (int)T, (int)tc_tiles, (int)it.num_pages, (int)ps, (int)nh, (int)nkv,
                                                      (int)hd, scale, (int)L.window, s.err, s.stream),
                   "attention_tc");
                return o;
            }
        }
        // How many CTAs share the keys of one tile: enough to fill the GPU when the batch alone does not, but at
        // least two blocks of 64 keys each.
        const bool wide = s.max_q_len * G > 16;
        const i64 bm = wide ? 64 : 16;
        i64 n_tiles = 0;
        for (i64 b = 0; b < s.B; ++b) n_tiles += ceil_div(s.q_lens[b] * G, bm);
        const i64 blocks = ceil_div(s.max_total_len, 64);
        const i64 target = ceil_div(4 * p.sms, n_tiles * nkv);
        const i64 nsplit = std::max<i64>(1, std::min(target, blocks / 2));
        void *part_o = nullptr, *part_ml = nullptr;
        if (nsplit > 1) {
            const i64 rows = T * nh;
            need_attn_ws = std::max(need_attn_ws, nsplit * rows * (hd + 2));
            if (!dry && nsplit * rows * (hd + 2) > s.attn_ws_floats) throw std::runtime_error("executor: the attention workspace is too small");
            part_o = s.attn_ws;
            part_ml = (float*)s.attn_ws + nsplit * rows * hd;
        }
        LAUNCH(fn<AttentionFlashFn>(FN_ATTENTION_FLASH)(o, part_o, part_ml, q, it.k, it.v, s.cu_seqlens, s.ctx_lens, it.block_table,
                                                    (int)it.bt_stride, (int)s.B, (int)T, (int)n_tiles, (int)it.num_pages, (int)ps,
                                                    (int)nh, (int)nkv, (int)hd, scale, (int)L.window, wide ? 1 : 0, (int)nsplit,
                                                    s.err, s.stream),
           "attention_flash");
        if (nsplit > 1) ++launches;                    // the merge of the pieces
        return o;
    }
    // 32-bit, other head sizes: one block per (token, head) over the block table
    if (hdv != hd) {
        LAUNCH(fn<AttentionPlainFn>(FN_ATTENTION_PLAIN_WIDE)(o, q, it.k, it.v, s.positions, s.seq_of_token, it.block_table, (int)it.bt_stride,
                                                         (int)it.num_pages, (int)it.page_size, (int)T, (int)nh, (int)nkv, (int)hd, (int)hdv,
                                                         scale, (int)L.window, (int)act, s.err, s.stream),
               "attention_plain_wide");
        return o;
    }
    LAUNCH(fn<AttentionPlainFn>(FN_ATTENTION_PLAIN)(o, q, it.k, it.v, s.positions, s.seq_of_token, it.block_table, (int)it.bt_stride,
                                                (int)it.num_pages, (int)it.page_size, (int)T, (int)nh, (int)nkv, (int)hd, (int)hd, scale,
                                                (int)L.window, (int)act, s.err, s.stream),
       "attention_plain");
    return o;
}

void Run::attention(const AttentionParams& L, const ExecItem& it, const void* x, void* out) {
    const i64 T = s.T, H = p.H, nh = L.nh, hd = L.hd;
    const i64 nkv = it.writes ? L.nkv : 0;
    void* q = nullptr;
    const i64 hdv = L.hdv > 0 ? L.hdv : hd;
    if (hdv != hd || L.norm_whole || L.temp_coef != 0.0 || L.pad) {
        // the general form: values of a width of their own, a norm over the whole projection, a query temperature
        if (L.rot || L.inv_freq) throw std::runtime_error("executor: the general attention form has no rotation");
        if (L.pad && (L.pad < hd || L.pad < hdv)) throw std::runtime_error("executor: heads padded to less than their width");
        const i64 width = nh * hd + nkv * (hd + hdv), hq = L.pad ? L.pad : hd, hv = L.pad ? L.pad : hdv;
        void* qkv = linear(x, L.qkv, T, H, act, width);       // without a cache of its own: the query rows only
        q = arena.take(T * nh * hq * elt(act));
        const int span = L.q_norm_w ? (L.norm_whole ? 2 : 1) : 0;
        LAUNCH(fn<AttnPrepFn>(FN_ATTN_PREP)(q, qkv, width, L.q_norm_w, L.k_norm_w, L.q_norm_w ? (int)L.qk_dtype : 0, (float)L.qk_eps, span,
                                        (float)L.temp_coef, (int)L.temp_every, s.positions, s.seq_of_token,
                                        nkv ? it.block_table : nullptr, nkv ? (int)it.bt_stride : 0, nkv ? it.k : nullptr,
                                        nkv ? it.v : nullptr, nkv ? (int)it.num_pages : 0, (int)it.page_size, (int)T, (int)nh, (int)nkv,
                                        (int)hd, (int)hdv, (int)hq, (int)hv, (int)act, s.err, s.stream),
               "attn_prep");
        if (L.pad) {        // from here on an ordinary attention with heads of the padded width
            AttentionParams P = L;
            P.hd = L.pad;
            P.hdv = 0;
            void* o = attend(P, it, q);
            product(out, o, L.out_proj, T, nh * L.pad, act);
            return;
        }
        void* o = attend(L, it, q);
        product(out, o, L.out_proj, T, nh * hdv, act);
        return;
    }
    // decode steps, bfloat16, heads of 64 turned whole in the "half" layout, a cache of the item's own: the product,
    // the heads' norm, the rotation and the cache write as one kernel
    const bool rope_fused = p.fused_rope && s.max_q_len == 1 && it.writes && hd == 64 && act == EXEC_BF16 &&
                            L.qkv.dtype == EXEC_BF16 && L.q_norm_w && L.qk_dtype == EXEC_BF16 && L.rot == 64 && !L.interleaved &&
                            L.inv_freq && tc_ok(L.qkv, H);
    i64 bn, split;
    if (rope_fused && epilogue_plan(T, (nh + 2 * nkv) * hd, H, &bn, &split)) {
        q = arena.take(T * nh * hd * elt(act));
        LAUNCH(fn<GemmRopeFn>(FN_GEMM_ROPE)(q, x, L.qkv.w, (int)T, (int)H, H, L.qkv.ldw, (int)bn, (int)split, L.q_norm_w, L.k_norm_w,
                                        (float)L.qk_eps, s.positions, it.block_table, (int)it.bt_stride, it.k, it.v,
                                        (int)it.num_pages, (int)it.page_size, (int)nh, (int)nkv, L.inv_freq, (int)p.static_flag,
                                        s.err, s.stream),
           "gemm_rope_tcgen05");
    } else {
        const i64 width = (nh + 2 * nkv) * hd;
        void* qkv = linear(x, L.qkv, T, H, act, width);       // without a cache of its own: the query rows only
        q = arena.take(T * nh * hd * elt(act));
        LAUNCH(fn<QkNormRopeFn>(FN_QK_NORM_ROPE)(q, qkv, width, L.q_norm_w, L.k_norm_w, L.q_norm_w ? (int)L.qk_dtype : 0,
                                             (float)L.qk_eps, s.positions, s.seq_of_token, nkv ? it.block_table : nullptr,
                                             nkv ? (int)it.bt_stride : 0, nkv ? it.k : nullptr, nkv ? it.v : nullptr,
                                             nkv ? (int)it.num_pages : 0, (int)it.page_size, (int)T, (int)nh, (int)nkv, (int)hd,
                                             (int)L.rot, (int)L.interleaved, L.inv_freq, (int)act, s.err, s.stream),
           "qk_norm_rope");
    }
    void* o = attend(L, it, q);
    product(out, o, L.out_proj, T, nh * hd, act);
}

void Run::gated_mlp(const GatedMlpParams& L, const void* x, void* out) {
    const i64 T = s.T, H = p.H;
    // gate and up stay 32-bit until act(g) * u is formed; the way back takes its bias before it is rounded
    void* gu = linear(x, L.gate_up, T, H, EXEC_F32);
    void* h = arena.take(T * L.ff * elt(act));
    if (L.extra) gate_at = static_cast<const float*>(gu) + 2 * L.ff, gate_ld = L.gate_up.N, gate_dtype = EXEC_F32;
    LAUNCH(fn<GatedActFn>(FN_GATED_ACT)(h, gu, L.gate_up.N, L.bg, L.bu, (int)L.b_dtype, (int)T, (int)L.ff, (int)L.act, (int)act, (int)EXEC_F32, s.stream),
           "gated_act");
    if (L.bd && may_leave_bias) {
        product(out, h, L.down, T, L.ff, act);
        pending_bias = L.bd;
    } else if (L.bd) {
        void* sums = linear(h, L.down, T, L.ff, EXEC_F32);
        LAUNCH(fn<BiasAddFn>(FN_BIAS_ADD)(out, sums, L.bd, (int)L.b_dtype, (int)T, (int)L.down.N, (int)act, s.stream), "bias_add");
    } else {
        product(out, h, L.down, T, L.ff, act);
    }
}

void Run::routed_mlp(const RoutedMlpParams& L, const void* x, void* out) {
    const i64 T = s.T, H = p.H, e = elt(act);
    if (L.up.dtype != act || L.down.dtype != act || L.router.dtype != act)
        throw std::runtime_error("executor: experts whose element type differs from the activations'");
    void* idx = arena.take(T * L.top * 4);
    void* wts = arena.take(T * L.top * 4);
    void* gate = L.shared_gate ? arena.take(T * 4) : nullptr;
    // the router's sums (and the shared expert's gate, one row more of the same matrix) as a product with 32-bit output
    void* z = linear(x, L.router, T, H, EXEC_F32);
    LAUNCH(fn<RouteFn>(FN_ROUTE)(idx, wts, gate, z, L.router.N, L.correction, (int)L.c_dtype, (int)T, (int)L.experts, (int)L.top,
                             (int)L.n_groups, (int)L.keep, (float)L.scale, L.shared_gate ? 1 : 0, s.stream),
           "route");
    const bool grouped = act == EXEC_BF16 && T >= p.grouped_min_tokens && tc_ok(L.up, H) && tc_ok(L.down, L.ff) && (((uintptr_t)x) & 15) == 0;
    if (!grouped) {
        // few tokens (and 32-bit): every token's chosen experts, and the shared one as one expert more, walked row by row
        void* mid = arena.take(T * L.top * L.ff * e);
        void* smid = L.shared_up.w ? arena.take(T * L.shared_ff * e) : nullptr;
        LAUNCH(fn<ExpertsRowwiseFn>(FN_EXPERTS_ROWWISE)(out, mid, smid, x, H, L.up.w, L.down.w, L.shared_up.w, L.shared_down.w, idx, wts, gate,
                                                    (int)T, (int)H, (int)L.ff, (int)L.shared_ff, (int)L.top, (int)L.experts, (int)L.act,
                                                    (int)act, s.stream),
               "experts_rowwise");
        ++launches;         // up and down are a launch each
        return;
    }
    // the shared expert: two plain products around its activation; its result stays 32-bit until the experts' sum takes it
    void* shared = nullptr;
    if (L.shared_up.w) {
        void* h = arena.take(T * L.shared_ff * e);
        if (tc_ok(L.shared_up, H)) {        // the activation on the 32-bit sums in the product's epilogue
            LAUNCH(fn<GemmGroupedFn>(FN_GEMM_GROUPED)(h, x, L.shared_up.w, (int)T, (int)L.shared_ff, (int)H, 1, H, L.shared_up.ldw, L.shared_ff,
                                                  (int)EXEC_BF16, nullptr, (int)L.act, s.err, s.stream),
                   "gemm_grouped_tcgen05");
        } else {
            void* u = linear(x, L.shared_up, T, H, EXEC_F32);
            LAUNCH(fn<ActivationFn>(FN_ACTIVATION)(h, u, L.shared_ff, (int)T, (int)L.shared_ff, (int)L.act, (int)act, s.stream), "activation");
        }
        shared = linear(h, L.shared_down, T, L.shared_ff, EXEC_F32);
    }
    {
        // many tokens: the slots sorted by expert, every expert's run padded to whole tiles of 128 rows, and the two
        // products as grouped tensor-core products over the sorted rows (the activation in the first one's epilogue)
        const i64 S = T * L.top, rows = ceil_div(S + std::min(L.experts, S) * 127, 128) * 128, tiles = rows / 128;
        void* row_slot = arena.take(rows * 4);
        void* slot_row = arena.take(S * 4);
        void* tile_group = arena.take(tiles * 4);
        LAUNCH(fn<MoeSortFn>(FN_MOE_SORT)(row_slot, slot_row, tile_group, idx, (int)S, (int)L.experts, (int)tiles, s.stream), "moe_sort");
        void* xs = arena.take(rows * H * 2);
        LAUNCH(fn<MoeGatherFn>(FN_MOE_GATHER)(xs, x, H, row_slot, tile_group, (int)rows, (int)L.top, (int)H, s.stream), "moe_gather");
        void* mid = arena.take(rows * L.ff * 2);
        LAUNCH(fn<GemmGroupedFn>(FN_GEMM_GROUPED)(mid, xs, L.up.w, (int)rows, (int)L.ff, (int)H, (int)L.experts, H, L.up.ldw, L.ff, (int)EXEC_BF16,
                                              tile_group, (int)L.act, s.err, s.stream),
               "gemm_grouped_tcgen05");
        void* ys = arena.take(rows * H * 2);
        LAUNCH(fn<GemmGroupedFn>(FN_GEMM_GROUPED)(ys, mid, L.down.w, (int)rows, (int)H, (int)L.ff, (int)L.experts, L.ff, L.down.ldw, H,
                                              (int)EXEC_BF16, tile_group, -1, s.err, s.stream),
               "gemm_grouped_tcgen05");
        LAUNCH(fn<MoeCombineFn>(FN_MOE_COMBINE)(out, ys, slot_row, wts, shared, gate, (int)T, (int)H, (int)L.top, s.stream), "moe_combine");
    }
}

void Run::mingru(const MinGruParams& L, const ExecItem& it, const void* x, void* out) {
    const i64 T = s.T, H = p.H, W = L.width;
    if (!it.state) throw std::runtime_error("executor: a recurrent mixer without a state slot");
    // the three projections side by side as 32-bit sums: what enters the recurrence is formed from them unrounded (a
    // rounding of z would be carried along by the state)
    void* proj = linear(x, L.in_proj, T, H, EXEC_F32);
    void* y = arena.take(T * W * elt(act));
    if (L.extra) gate_at = static_cast<const float*>(proj) + 3 * W, gate_ld = L.in_proj.N, gate_dtype = EXEC_F32;
    LAUNCH(fn<MinGruScanFn>(FN_MINGRU_SCAN)(y, proj, L.in_proj.N, (int)EXEC_F32, L.bz, L.bx, (int)L.b_dtype, it.state, it.slot_stride, s.slot_ids,
                                        s.cu_seqlens, (int)T, (int)s.B, (int)W, (int)it.n_slots, (int)s.max_q_len, (int)act, s.err, s.stream),
           "mingru_scan");
    product(out, y, L.out_proj, T, W, act);
}

void Run::latent_attention(const LatentAttentionParams& L, const ExecItem& it, const void* x, void* out) {
    const i64 T = s.T, H = p.H, nh = L.heads, kw = L.rank + L.rot_dim, e = elt(act);
    void* proj = linear(x, L.in_proj, T, H, act);
    if (L.extra) gate_at = static_cast<const char*>(proj) + (L.in_proj.N - L.extra) * e, gate_ld = L.in_proj.N, gate_dtype = act;
    void* q_plain = arena.take(T * nh * L.dim * e);
    void* q_full = arena.take(T * nh * kw * e);
    LAUNCH(fn<LatentPrepFn>(FN_LATENT_PREP)(q_plain, q_full, proj, L.in_proj.N, (int)act, L.c_norm_w, (int)L.c_norm_dtype, (float)L.eps,
                                        s.positions, s.seq_of_token, it.block_table, (int)it.bt_stride, it.writes ? it.k : nullptr,
                                        (int)it.num_pages, (int)it.page_size, (int)T, (int)nh, (int)L.dim, (int)L.rot_dim, (int)L.rank,
                                        (int)L.rot, (int)L.interleaved, L.inv_freq, (int)act, s.err, s.stream),
           "latent_prep");
    // a head's query against the cached rows: [K_h^T q_h | rotated part]
    head_products(q_full, nh * kw, kw, q_plain, nh * L.dim, L.dim, L.absorb_k, T, nh, L.rank, L.dim);
    // every head reads the same rows (one key/value head); a value is a row's first `rank` entries
    void* o_lat = arena.take(T * nh * L.rank * e);
    // bfloat16 and sizes the tensor-core kernel takes (multiples of 16, value columns that split over its warps, tiles
    // that fit shared memory): 64 (token, head) rows a CTA; the keys in pieces when the tiles alone leave SMs idle
    i64 dvw = 0;
    if (L.rank % 256 == 0 && L.rank / 256 <= 2) dvw = 256;
    else if (L.rank % 128 == 0 && L.rank / 128 <= 4) dvw = 128;
    else if (L.rank % 64 == 0 && L.rank / 64 <= 4) dvw = 64;
    else if (L.rank % 32 == 0 && L.rank / 32 <= 8) dvw = 32;
    else if (L.rank % 16 == 0 && L.rank / 16 <= 8) dvw = 16;
    const i64 bn = dvw == 256 ? ((64 + 128) * (kw + 8) * 2 + 2048 <= 227 * 1024 ? 64 : 32) : (dvw == 64 ? 64 : 32);
    if (p.latent_tc && act == EXEC_BF16 && L.scale > 0 && dvw && kw % 16 == 0 && (64 + 2 * bn) * (kw + 8) * 2 + 2048 <= 227 * 1024) {
        i64 n_tiles = 0;
        for (i64 b = 0; b < s.B; ++b) n_tiles += ceil_div(s.q_lens[b] * nh, 64);
        const i64 blocks = ceil_div(L.window ? std::min<i64>(s.max_total_len, L.window + s.max_q_len) : s.max_total_len, bn);
        // pieces of the keys: what fills the SMs once (two CTAs an SM where two tiles of this width fit its shared
        // memory), of at least two blocks of keys each
        const i64 per_sm = std::min<i64>(2, std::max<i64>(1, 227 * 1024 / ((64 + 2 * bn) * (kw + 8) * 2)));
        // (rounded down: one CTA more than the SMs hold at once would wait for a second round by itself)
        const i64 nsplit = std::max<i64>(1, std::min(per_sm * p.sms / n_tiles, blocks / 2));
        void *part_o = nullptr, *part_ml = nullptr;
        if (nsplit > 1) {
            const i64 rows = T * nh;
            need_attn_ws = std::max(need_attn_ws, nsplit * rows * (L.rank + 2));
            if (!dry && nsplit * rows * (L.rank + 2) > s.attn_ws_floats) throw std::runtime_error("executor: the attention workspace is too small");
            part_o = s.attn_ws;
            part_ml = (float*)s.attn_ws + nsplit * rows * L.rank;
        }
        LAUNCH(fn<AttentionLatentFn>(FN_ATTENTION_LATENT)(o_lat, part_o, part_ml, q_full, it.k, s.cu_seqlens, s.ctx_lens, it.block_table,
                                                      (int)it.bt_stride, (int)s.B, (int)T, (int)n_tiles, (int)it.num_pages,
                                                      (int)it.page_size, (int)nh, (int)kw, (int)L.rank, (float)L.scale, (int)nsplit,
                                                      (int)L.window, L.sinks, s.err, s.stream),
               "attention_latent");
        if (nsplit > 1) ++launches;                    // the merge of the pieces
    } else if (L.window || L.sinks)
    LAUNCH(fn<AttentionPlainMaskedFn>(FN_ATTENTION_PLAIN_MASKED)(o_lat, q_full, it.k, it.k, s.positions, s.seq_of_token, it.block_table,
                                                             (int)it.bt_stride, (int)it.num_pages, (int)it.page_size, (int)T, (int)nh, 1,
                                                             (int)kw, (int)L.rank, (int)kw, (float)L.scale, (int)L.window, 0, L.sinks, 0.f, 0,
                                                             nullptr, 0, (int)act, s.err, s.stream),
           "attention_plain_masked");
    else
    LAUNCH(fn<AttentionPlainFn>(FN_ATTENTION_PLAIN)(o_lat, q_full, it.k, it.k, s.positions, s.seq_of_token, it.block_table, (int)it.bt_stride,
                                                (int)it.num_pages, (int)it.page_size, (int)T, (int)nh, 1, (int)kw, (int)L.rank,
                                                (float)L.scale, 0, (int)act, s.err, s.stream),
           "attention_plain");
    void* o = arena.take(T * nh * L.vdim * e);
    head_products(o, nh * L.vdim, L.vdim, o_lat, nh * L.rank, L.rank, L.expand_v, T, nh, L.vdim, L.rank);
    product(out, o, L.out_proj, T, nh * L.vdim, act);
}

int walk(const ExecProgram& p, ExecStep& s, bool dry, i64* need) {
    Run r{p, s, Arena{static_cast<char*>(s.arena), s.arena_bytes}, p.act_dtype};
    r.dry = r.arena.dry = dry;
    if (dry) r.arena.base = reinterpret_cast<char*>(4096);     // sizes only: addresses that are never used, but not null
    const i64 T = s.T, H = p.H, e = elt(p.act_dtype);
    s.launches = 0;
    for (i64& c : s.calls) c = 0;
    if (T <= 0) return 0;
    if (s.n_order > p.n_order) throw std::runtime_error("executor: more order items than the program has");
    r.regs.x = r.arena.take(T * H * 4);
    r.slot[0] = r.arena.take(T * H * e);
    r.slot[1] = r.arena.take(T * H * e);
    r.arena.keep();
    r.regs.phase = 0;
    r.run(p.prologue);
    r.regs.phase = 1;
    for (i64 i = 0; i < s.n_order; ++i) {
        const i64 layer = p.order[i];
        if (layer < 0 || layer >= p.n_layers) throw std::runtime_error("executor: the run order names a layer the program lacks");
        r.regs.item = i;
        r.run(p.layers[layer]);
    }
    if (s.R > 0) {
        r.regs.phase = 2;
        r.regs.logits = s.logits;
        r.run(p.epilogue);
    }
    s.launches = r.launches;
    if (need) { need[0] = r.arena.peak; need[1] = r.need_gemm_ws; need[2] = r.need_attn_ws; }
    return 0;
}
}  // namespace

int exec_forward(const ExecProgram& p, ExecStep& s) { return walk(p, s, false, nullptr); }

void exec_need(const ExecProgram& p, ExecStep& s, i64* need) { walk(p, s, true, need); }

int exec_part(const ExecProgram& p, ExecStep& s, const ExecOp& op, const void* y_in, void* out, bool dry, i64* need) {
    Run r{p, s, Arena{static_cast<char*>(s.arena), s.arena_bytes}, p.act_dtype};
    r.dry = r.arena.dry = dry;
    if (dry) r.arena.base = reinterpret_cast<char*>(4096);     // sizes only: addresses that are never used, but not null
    s.launches = 0;
    for (i64& c : s.calls) c = 0;
    if (s.T > 0) {
        r.regs.phase = 1;
        r.produce(op, s.items, y_in, out);
    }
    s.launches = r.launches;
    if (need) { need[0] = r.arena.peak; need[1] = r.need_gemm_ws; need[2] = r.need_attn_ws; }
    return 0;
}

}  // namespace cellm
