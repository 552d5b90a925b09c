// The forward pass of one step, launched from native code.
//
// A model is described to the executor as a program of op records: a prologue
// (the embedding), the records of every layer, the run order of the layers, and
// an epilogue (final norm on the wanted rows, output product). The records are
// emitted by the parts themselves (cellm_b200/parts: each part's emit()), one
// record per part, so the executor knows kinds of parts, never a model: a layer
// is whatever list of records its block arrangement emitted. A part that has no
// native record emits OP_PYTHON, and the executor calls back into the
// interpreter for that part alone; the parts around it stay native.
//
// The records work on three registers:
//   x        the 32-bit residual stream [T, H]
//   pending  an addend [T, H] that waits to be added into x (or null)
//   y        the activations the next part reads (the output of the last norm)
// A norm adds `pending` into x and leaves the normed rows in y; a mixer or a
// feed-forward reads y and leaves its output as the new `pending` (if one waits
// already, that one is added into x first).
//
// The executor also owns the decisions below the parts: which kernel serves a
// product or an attention of a given shape, which tile shape and K split. The
// interpreter's kernel wrappers ask it (cellm_exec_plan_tiles, cellm_exec_part)
// instead of deciding a second time.
//
// The kernels are reached through a table of entry points that the caller fills
// (the addresses of the compiled libraries' C symbols), so this file has no
// dependency on CUDA and its decisions can be tested on a machine without a GPU
// by filling the table with recording stand-ins.
//
// All structs have 8-byte fields only, so that their layout is the same on both
// sides of the foreign call; cellm_exec_sizeof() lets the caller check.
#pragma once
#include <cstdint>

namespace cellm {

typedef long long i64;

// Element types as the kernels tag them.
enum : i64 { EXEC_F32 = 0, EXEC_BF16 = 1 };

struct ExecLinear {
    const void* w;      // [N, K], row pitch ldw elements
    i64 N, K, ldw;
    i64 dtype;          // element type of w
    i64 tc_ok;          // w meets the tensor-core kernel's alignment rules
};

// ---- op records ---------------------------------------------------------------------------------------------------
enum OpKind : i64 {
    OP_EMBED = 0, OP_RMS_NORM, OP_SHORT_CONV, OP_ATTENTION, OP_SWIGLU, OP_HEAD, OP_PYTHON,
    // pieces of the above by themselves, for exec_part only (the interpreter's kernel wrappers)
    OP_LINEAR, OP_ATTEND,
    // a layer whose sublayers read the stream itself and whose results join it through a gate and a norm
    OP_READ_STREAM, OP_GATED_NORM_ADD, OP_MINGRU, OP_LATENT_ATTENTION, OP_GATED_MLP,
    // a feed-forward whose tokens each run a few of many small experts, chosen by a router
    OP_ROUTED_MLP, OP_KINDS
};

struct ExecOp {
    i64 kind;
    const void* params;     // the kind's parameter struct below
};

// x = table[ids] * scale (+ pos_table[positions], learned position vectors [max_pos, H] of the table's element type; null: none)
struct EmbedParams { const void* table; i64 dtype; double scale; const void* pos_table; i64 max_pos; };
struct RmsNormParams { const void* w; i64 dtype; double eps; i64 groups; };   // x += pending; y = rms_norm(x) * w (the mean over each of `groups` parts)
struct ShortConvParams {
    ExecLinear in_proj, out_proj;
    const void* in_proj_tiled; i64 tiled_rows;      // in_proj in tiles of 42 channels for the fused decode kernel (null: none)
    const void* taps; const void* bias; i64 taps_dtype, n_taps;
};
struct AttentionParams {
    ExecLinear qkv, out_proj;
    i64 nh, nkv, hd, window; double scale;
    const void* q_norm_w; const void* k_norm_w; i64 qk_dtype; double qk_eps;
    i64 rot, interleaved; const void* inv_freq;     // rot = 0 with inv_freq null: no rotation
    // The general form (attn_prep.cu), taken when any of these differs from its default; it has no rotation.
    i64 hdv;                // width of a value head (0: hd); the item's pool of values has rows of this width
    i64 norm_whole;         // 1: q and k are normed over all their heads at once (weights [nh * hd], [nkv * hd]); 0: per head
    double temp_coef; i64 temp_every;       // q *= 1 + temp_coef * ln(floor((pos + 1) / temp_every) + 1); coef 0: none
    i64 pad;                // > 0: queries, keys and values are kept in heads of this width, zeros behind their own entries, so that
                            // the attention is an ordinary one of that head size; out_proj then has nh * pad columns
};
struct SwiGLUParams {
    ExecLinear gate_up, down;
    i64 ff, fused;      // fused: gate_up holds interleaved gate and up blocks for the product's SwiGLU epilogue
};
struct HeadParams { ExecLinear w; };                                   // logits = y . w^T in 32-bit
struct PythonParams { i64 token; };                                    // the interpreter's name for the part
struct LinearParams { ExecLinear w; i64 lda, out_dtype; };             // out [T, N] = in [T, K] (row pitch lda) . w^T
// OP_ATTEND takes AttentionParams and reads only nh, nkv, hd, window and scale: out = attention of the queries `in`
// [T, nh * hd] (normed, turned) over the item's pages.

// y = x in the activations' element type (a pending addend goes into x first): the input of a sublayer that reads the
// stream itself. Nothing is launched when y already holds x.
struct ReadStreamParams { i64 reserved; };
// x += group_rms_norm(pending * sigmoid(y . gate^T + gate_bias)) * w, then y = x: a sublayer's result joins the stream.
// gate.w null: no gate. y is the sublayer's input when the record starts.
// stacked: the gate's rows lie behind the rows of the sublayer's own first product (its `extra`), which has formed the gate already.
struct GatedNormAddParams { ExecLinear gate; const void* gate_bias; const void* w; i64 w_dtype, groups; double eps; i64 stacked; };
// minGRU: in_proj stacks the rows of z, candidate and output gate ([3 * width, H]); the state is the item's slot [width].
// `extra` (here and below): rows stacked behind the part's own in its first matrix, whose products the part leaves for the
// record after it (a gate over the same input).
struct MinGruParams { ExecLinear in_proj, out_proj; const void* bz; const void* bx; i64 b_dtype, width, extra; };
// Latent attention: in_proj stacks the queries' rows (heads * (dim + rot_dim)), the latent's (rank) and the shared
// rotated key part's (rot_dim). absorb_k: [heads, rank, dim] (a head's key matrix transposed), expand_v: [heads, vdim,
// rank]. The item's pages hold rows of rank + rot_dim values.
struct LatentAttentionParams {
    ExecLinear in_proj, out_proj;
    const void* absorb_k; const void* expand_v;
    i64 heads, dim, rot_dim, vdim, rank; double scale;
    const void* c_norm_w; i64 c_norm_dtype; double eps;
    i64 rot; const void* inv_freq;
    i64 extra;
    i64 interleaved;            // the rotation's pairs: (2p, 2p + 1), or (p, p + rot / 2)
    i64 window;                 // 0: every earlier row; w: a token reads its last w rows
    const void* sinks;          // [heads] 32-bit: one more term exp(sink_h) in a head's denominator; null: none
};
// down . (act(gate . y + bg) * (up . y + bu)) + bd; act 0 silu, 1 gelu (tanh form); the biases may be null.
struct GatedMlpParams { ExecLinear gate_up, down; const void* bg; const void* bu; const void* bd; i64 b_dtype, ff, act, extra; };

// Routed experts: out = sum over the token's `top` chosen experts of weight * down_e act(up_e y) (+ sigmoid(g . y) * shared(y)).
// up: [experts * ff, H] and down: [experts * H, ff], the experts' matrices one below the other. router: [experts (+ 1), H], the
// last row the shared expert's gate when it has one. The choice: see routed.cu. act: 0 gelu (erf), 1 gelu (tanh), 2 silu, 3 relu.
struct RoutedMlpParams {
    ExecLinear up, down, router;
    const void* correction; i64 c_dtype;
    i64 experts, top, n_groups, keep; double scale;
    i64 ff, act;
    ExecLinear shared_up, shared_down;      // w null: no shared expert
    i64 shared_ff, shared_gate;
};

struct ExecOps { i64 n; const ExecOp* ops; };

// The registers as a Python part sees and changes them.
struct ExecRegs {
    void* x;
    const void* pending;
    void* y;
    void* logits;       // [R, V] float, epilogue only
    i64 phase;          // 0 prologue, 1 layers, 2 epilogue (rows = the wanted rows only)
    i64 item;           // index in the run order (phase 1)
};
// Runs the part `token`; may replace pending and y. Returns 0, or non-zero after an error the caller keeps.
typedef i64 (*PythonOpFn)(i64 token, ExecRegs* regs);

// Entry points of the kernel libraries, in the order of ExecProgram::fns.
enum ExecFn {
    FN_EMBED, FN_ADD_RMSNORM, FN_RESIDUAL_ADD, FN_SWIGLU, FN_SHORT_CONV, FN_QK_NORM_ROPE, FN_ATTENTION_PLAIN, FN_GEMM_PLAIN,
    FN_ATTENTION_DECODE, FN_ATTENTION_TC, FN_ATTENTION_FLASH, FN_GEMM_TCGEN05, FN_GEMM_CONV, FN_GEMM_ROPE,
    FN_GATED_NORM_ADD, FN_STREAM_CAST, FN_MINGRU_SCAN, FN_LATENT_PREP, FN_HEAD_PRODUCT, FN_GATED_ACT, FN_BIAS_ADD, FN_ATTENTION_LATENT, FN_HEAD_PRODUCT_MMA,
    FN_EMBED_POS, FN_ATTN_PREP, FN_ATTENTION_PLAIN_WIDE, FN_ROUTE, FN_EXPERTS_ROWWISE, FN_ACTIVATION, FN_ADD2_RMSNORM,
    FN_MOE_SORT, FN_MOE_GATHER, FN_MOE_COMBINE, FN_GEMM_GROUPED, FN_ATTENTION_PLAIN_MASKED, FN_COUNT
};

struct ExecProgram {
    i64 n_layers, n_order, H, V, act_dtype;
    i64 sms, static_flag, max_counters;
    i64 fused_conv, fused_rope;     // decode steps: in_proj + convolution, q/k/v product + norm + rotation as one kernel each
    i64 latent_tc;                  // latent attention on the tensor cores where its sizes allow (0: the plain kernel always)
    i64 grouped_min_tokens;         // routed experts run as grouped tensor-core products from this many tokens (bfloat16)
    i64 tc_min_ctas;                // prompt attention on tcgen05 from this many CTAs (< 0: an eighth of the SMs)
    double tc_min_fill;             // and this share of its tiles' rows in use
    ExecOps prologue, epilogue;
    const ExecOps* layers;          // [n_layers]
    const i64* order;               // [n_order]: the layer each item of the run order runs
    PythonOpFn python;
    void* fns[FN_COUNT];
};

// The cache an item of the run order works on in this step.
struct ExecItem {
    void* k; void* v; const void* block_table;
    i64 bt_stride, num_pages, page_size, writes;
    void* state; i64 slot_stride, n_slots;
};

struct ExecStep {
    i64 T, B, R, max_q_len, max_total_len, n_order;   // n_order: run only the first items (<= program's)
    const void *ids, *positions, *seq_of_token, *cu_seqlens, *ctx_lens, *slot_ids, *rows;
    const i64* q_lens;          // host copy, [B]
    const ExecItem* items;      // [n_order]
    void* arena; i64 arena_bytes;
    void* logits;               // [R, V] float, or null when R = 0
    void* err; void* stream;
    void* gemm_ws; i64 gemm_ws_floats;
    void* attn_ws; i64 attn_ws_floats;
    void* counters;
    i64 launches;               // out: kernels launched by native records
    i64 calls[FN_COUNT];        // out: calls of each entry point
};

// What the step needs, found by walking it without a launch: need[0] bytes of arena, need[1] floats of
// the products' workspace, need[2] floats of the attention workspace. Also sets s.launches.
void exec_need(const ExecProgram& p, ExecStep& s, i64* need);
// Runs the step. 0, or throws with the failing kernel's status in the message.
int exec_forward(const ExecProgram& p, ExecStep& s);
// One record of a mixer or feed-forward (or OP_LINEAR, OP_ATTEND) by itself: reads y_in, writes out (for a mixer or
// feed-forward both [T, H] of the activations' element type); the cache is s.items[0]. With dry set nothing is launched and need[] is filled as by exec_need.
int exec_part(const ExecProgram& p, ExecStep& s, const ExecOp& op, const void* y_in, void* out, bool dry, i64* need);

// The tile shape and K split of a product of M tokens by N weight rows over K.
void plan_tiles(i64 M, i64 N, i64 K, i64 sms, i64* bn, i64* split);

}  // namespace cellm
