// Kernels for models that run a RAGGED BATCH per step: the rows of one step are portions of several sequences (a prompt
// chunk of one beside single decoded tokens of others), concatenated, with per-row and per-entry descriptors in device memory.
// Every mechanism takes its constants as arguments so that any layer-list model can be assembled from them:
//   Dynamic-Tanh norm, RMS norm with up to two weights on one statistic, RMS QK norm (weightless or weighted) with a
//   position-dependent query temperature and / or an interleaved-pair rotation of the leading dimensions, paged softmax attention
//   with a sink term, an optional sliding window and an optional sigmoid output gate
//   (any key width, any value width, grouped queries, keys / values optionally owned by another layer), the Mamba-2 mixer
//   (causal depthwise convolution with carried window, selective state-space scan with carried f32 state, gated grouped RMS
//   norm), a clamped gated feed-forward, and a mixture of experts (softmax or sigmoid scores, a selection bias, group-limited
//   choice, plain or gated experts, SiLU or clamped units, the score on the expert's input or output; router, counting sort, grouped
//   linears, ordered combine with a per-column scale, an every-token expert and a sigmoid gate).  See ragged.cu.  Further, in
//   ragged_mix.cu: a carried causal convolution in front of a sublayer, latent attention (one normalised low-rank row cached per
//   token), block-diagonal per-head linears, gated linear attention with a decay per key channel, a soft cap on logits.  For layers
//   whose sublayers read the stream itself and are normalised on their way back: a sinusoidal position vector on the embedding, the
//   post-norm residual add (one or two normalised inputs), attention scores with a tanh cap, a logarithmic distance penalty or a
//   distance table, projection biases, a whole-projection norm, unit-RMS values or values taken from the raw keys (ragged.cu), and,
//   in ragged_scan.cu, the Mamba-1 selective scan and the mLSTM matrix memory.
#pragma once

#include "common.cuh"

namespace cb {

struct RaggedBatch {
    const int* row_entry;   // [T] entry of each row
    const int* row_pos;     // [T] position of each row in its sequence (0-based)
    const int* ent_row0;    // [E] first row of the entry
    const int* ent_len;     // [E] rows of the entry
    const int* ent_pos0;    // [E] tokens the sequence held before this step
    const int* ent_slot;    // [E] sequence slot: block-table row and recurrent-state slot
    int T, E;
};

// An activation buffer as the linears read it: f32 rows (exact mode, routers) and / or bf16 planes hi (+ lo at an element offset).
struct ActOut {
    float* f = nullptr; int ldf = 0;
    bf16* hi = nullptr; long long lo_off = 0; int ldb = 0;
};

enum LinearMode : int { LIN_STORE = 0, LIN_RESID = 1 };

int embed_scale_rows_launch(cudaStream_t st, const int* ids, int T, const bf16* embed, int W, float scale, float* x, int ldx);
// x[r, c] = embed[ids[r], c] + (c even ? sin : cos)(row_pos[r] * freq[c / 2]): the embedding row plus a sinusoidal position vector.
// freq [ceil(W / 2)] radians per position; position and angle in f32
int embed_sinpos_rows_launch(cudaStream_t st, const int* ids, const int* row_pos, int T, const bf16* embed, int W, const float* freq, float* x, int ldx);
// Norm on a sublayer's way back into the stream.  One input: x[r] += rms(y1[r] + b1) * norm_w.  Two inputs (y2 != nullptr): each is
// RMS-normed with its own weight first and half their sum takes y1's place: v = (rms(y1 + b1) * w1 + rms(y2) * w2) / 2.
// b1, w1, w2 nullable.  Every mean of squares runs thread-strided, then over a fixed tree.  planes (optional): the new x also leaves as
// bf16 operand planes, for the linear that reads the stream next.
int post_norm_add_launch(cudaStream_t st, const float* y1, int ld1, const float* b1, const float* w1, const float* y2, int ld2, const float* w2,
                         const float* norm_w, float eps, float* x, int ldx, int T, int W, const ActOut& planes = ActOut{});
// out[r, c] = tanh(alpha * x[src(r), c]) * w[c] + b[c];  rows = gather list (nullptr: identity)
int dyt_rows_launch(cudaStream_t st, const float* x, int ldx, const int* rows, int R, int W, const float* alpha, const float* w,
                    const float* b, const ActOut& out);
// out_k[r, c] = x[src(r), c] / sqrt(mean_c(x^2) + eps) * w_k[c] for k = 1 and (optionally) 2: two norms of the same row share its
// statistic.  w_k holds the final multipliers (a weight stored around zero is registered as 1 + w).  groups > 1: the row is cut
// into that many equal consecutive parts, each divided by its own root mean square (W % groups == 0).  out1 may be x itself.
int rms_rows_launch(cudaStream_t st, const float* x, int ldx, const int* rows, int R, int W, float eps, const float* w1, const ActOut& out1,
                    const float* w2, const ActOut& out2, int groups = 1);
// dst[r, col0 + c] = src[r, c] for c < W, in every form dst carries (f32 rows, bf16 planes)
int store_rows_launch(cudaStream_t st, const float* src, int lds, int T, int W, const ActOut& dst, int col0);
// C[M, N] (+)= A[M, K] f32 x W[N, K]^T bf16, every product and sum in f32 (no tensor cores): the exact mode's linear, and the router's.
// col_scale (LIN_RESID only, nullable): C[m, n] += col_scale[n] * acc;  gate (LIN_RESID only, nullable [M, ldg], gate_bias nullable [N]):
// the added value is also multiplied by sigmoid(gate[m, n] + gate_bias[n])
int linear_f32_launch(cudaStream_t st, const float* A, int lda, const bf16* W, int ldw, int M, int N, int K, int mode, float* C, int ldc,
                      const float* col_scale = nullptr, const float* gate = nullptr, int ldg = 0, const float* gate_bias = nullptr);
// out[r, j] = silu(gu[r, 2j]) * gu[r, 2j + 1]  (interleaved (gate, up) pairs);  limit < 0: gelu_tanh in place of silu
int silu_glu_launch(cudaStream_t st, const float* gu, int ld, int T, int F, const ActOut& out, float limit = 0.f);

struct AttnPrepArgs {
    const float* qkv; int ld;         // [T, ld]: q heads | k heads | v heads (k / v absent when has_kv == 0)
    int H, G, d, dv;
    float eps;
    float temp_coef; int temp_every;  // temp_every <= 0: no query temperature
    const float* q_norm_w;            // [d] weights of the RMS norm of queries / keys, shared by the heads; nullptr = weightless
    const float* k_norm_w;
    int rot_dims;                     // > 0: after the norm, dimensions (2i, 2i + 1), i < rot_dims / 2, of q and k turn by pos * rot_freq[i]
    const double* rot_freq;           // [rot_dims / 2] radians per position (the angle and its sine / cosine are taken in 64-bit)
    ActOut q_out;                     // [T, H * d] normalised, temperature applied (f32 for sink_attention, planes for the flash kernel)
    void* k_pool; void* v_pool;       // pages [n_pages, G, KV_PAGE, d | dv] of f32, or of bf16 with an optional low-order plane
    int kv_f32; long long kv_lo_off;  // bf16 pages: element offset of the plane holding bf16(x - bf16(x)), 0 = none
    int has_kv;
    const int* block_table; int max_pages;
    int no_norm = 0;                  // 1: queries and keys pass as they are (no RMS norm, no temperature); rotation still applies
    const float* bias = nullptr;      // nullable [row width of qkv used]: added to every projected value before anything else
    int whole_norm = 0;               // 1: ONE RMS statistic over all query heads of the row (and one over all key heads); the norm
                                      //    weights then hold H * d (G * d) entries instead of d
    int v_unit = 0;                   // 1: every value head is divided by its root mean square over dv (eps, no weight) before it is cached
    int v_from_k = 0;                 // 1: the row has no value columns; the cached value of a head is its key as projected (+ bias), before the norm (dv == d)
    const float* q_head_scale = nullptr;   // nullable [H]: head h's normalised query is multiplied by q_head_scale[h]
};
int attn_prep_launch(cudaStream_t st, const RaggedBatch& rb, const AttnPrepArgs& a);

struct SinkAttnArgs {
    const float* q; int ldq;          // [T, H * d]
    const void* k_pool; const void* v_pool; int kv_f32; long long kv_lo_off;
    const int* block_table; int max_pages;
    int H, G, d, dv;
    float scale;
    const float* sink;                // [H] or nullptr (no sink term)
    int window;                       // > 0: row i sees keys j with 0 <= i - j < window; 0: every earlier key
    const float* gate; int ldg;       // nullable [T, ldg]: out[r, h * dv + c] *= sigmoid(gate[r, h * dv + c])
    ActOut out;                       // [T, H * dv]
    float* part; int nsplit;          // scratch [T, H, nsplit, dv + 2] when nsplit > 1
    int kv_shared = 0;                // 1: k_pool == v_pool and d == dv -- a cached row is its own value (staged once)
    // score modifiers, applied in this order after the scale: s <- softcap * tanh(s / softcap) (softcap > 0);
    // s <- s - dist_r1[h] * ln(1 + dist_r2[h] * (i - j)) (dist_r1 != nullptr);  s <- s + dist_table[h * dist_rows + min(i - j, dist_rows - 1)]
    float softcap = 0.f;
    const float* dist_r1 = nullptr; const float* dist_r2 = nullptr;
    const float* dist_table = nullptr; int dist_rows = 0;
};
int sink_attention_launch(cudaStream_t st, const RaggedBatch& rb, const SinkAttnArgs& a);

struct Mamba2Args {
    const float* proj; int ldp;       // [T, ldp]: z | x | B | C | dt
    int heads, P, N, groups, taps, norm_groups;
    const float* conv_w;              // [C, taps], C = heads * P + 2 * groups * N
    const float* conv_b;              // [C]
    const float* dt_bias; const float* A_log; const float* D;   // [heads]
    const float* norm_w;              // [heads * P]
    float eps;
    float* conv_state;                // [slots, taps - 1, C] the inputs before the next token
    float* ssm_state;                 // [slots, heads, N, P] f32
    float* xbc;                       // [T, C] scratch: conv + silu
    float* y;                         // [T, heads * P] scratch
    ActOut out;                       // gated, normalised [T, heads * P]
    int single_rows = 0;              // every entry brings exactly one row (a decode step): convolution and window shift fuse
    // long portions run as segments side by side (see ssd_scan_kernel): scratch for their local / start states and decay
    // products, mamba2_seg_floats(entries, ...) floats in all; nullptr = never segment
    float* seg_state = nullptr; float* seg_decay = nullptr;
    int max_len = 0;                  // rows of the longest entry
};
int mamba2_mixer_launch(cudaStream_t st, const RaggedBatch& rb, const Mamba2Args& a);
int mamba2_launch_count(bool single_rows, int max_len);
size_t mamba2_seg_floats(int entries, int heads, int N, int P);
size_t mamba2_seg_decay_offset(int entries, int heads, int N, int P);

// out[r, j] = g * sigmoid(1.702 g) * (u + 1),  g = min(gu[r, js], limit),  u = clamp(gu[r, js + up_off], -limit, limit),  js = j * stride
// (stride 2, up_off 1: interleaved (gate, up) pairs, the layout the fused GEMM / GEMV epilogues read)
int clamped_glu_launch(cudaStream_t st, const float* gu, int ld, int stride, int up_off, int T, int F, float limit, const ActOut& out);

struct MoeArgs {
    int T, E, top, F, W;              // rows, experts, experts per row, expert width, model width
    const float* h; int ldh;          // [T, ldh] f32 input rows
    float* router_logits; int ldr;    // [T, ldr]
    const bf16* const* up;            // [E] device pointers, each [F, ldwu]
    const bf16* const* down;          // [E] each [W, ldwd]
    int ldwu, ldwd;
    int* sel_e; float* sel_w;         // [T * top]
    int* sorted; int* tile_e; int* tile_r0; int* tile_n; int* n_tiles; int max_tiles;
    int* inv;                         // [T * top] place of each pair in `sorted`
    int* offs;                        // [E + 1] first place of each expert's pairs in `sorted`
    float* act; int lda;              // [T * top, lda]
    float* y; int ldy;                // [T * top, ldy]
    float* x; int ldx;                // residual, += out_scale * sum_k w_k y_k
    // selection: scores = softmax(logits) (score_fn 0) or sigmoid(logits) (1); the `top` experts with the largest score + correction
    // are chosen among the `keep` best of `n_groups` equal groups of neighbouring experts (a group's rank: the sum of its two largest
    // score + correction); the weights are the chosen experts' scores without the correction.  n_groups <= 1: no group limit.
    int score_fn = 0; const float* correction = nullptr; int n_groups = 0, keep = 0;
    int gated = 0;                    // 1: up[e] is [2F, ldwu] with (gate_j, up_j) rows interleaved, act = silu(gate) * up; 0: act = gelu_erf(up)
    const float* out_scale = nullptr; // [W] per-column factor of the combined output (nullptr: 1)
    float glu_limit = 0.f;            // gated experts: > 0 = the clamped unit min(g, L) * sigmoid(1.702 min(g, L)) * (clamp(u, -L, L) + 1)
    int scale_input = 0;              // 1: an expert reads weight * h (its output is summed unweighted) instead of having its output weighted
    int n_extra = 0; float* extra_out = nullptr;   // w_router carries n_extra (0 or 1) more rows behind the experts': extra_out[r] = sigmoid(row E . h)
    // the combine may also add an every-token expert and gate the sum:
    //   x[r, c] += sigmoid(gate[r, c] + gate_bias[c]) * out_scale[c] * (sum_k y_k[c] + shared_w[r] * shared_y[r, c])      (each part optional)
    const float* gate = nullptr; int ldg = 0; const float* gate_bias = nullptr;
    const float* shared_y = nullptr; int lds = 0; const float* shared_w = nullptr;
};
// router logits (f32 products: a.h x w_router^T -> a.router_logits), softmax + top-k, then the counting sort by expert
int moe_route_launch(cudaStream_t st, const MoeArgs& a, const bf16* w_router, int ldw);
// experts as grouped f32 linears over the sorted pairs + the ordered combine into x (3 launches): y rows indexed by pair
int moe_experts_launch(cudaStream_t st, const MoeArgs& a);
// tensor-core expert path: rows of `src` (bf16 planes) gathered into expert order, dense GEMMs per expert by the caller (y rows in
// sorted order), then the combine through `inv`
int moe_gather_launch(cudaStream_t st, const MoeArgs& a, const ActOut& src, const ActOut& dst);
int moe_combine_launch(cudaStream_t st, const MoeArgs& a, bool y_sorted);
inline int moe_max_tiles(int T, int top, int E) { return (T * top + 31) / 32 + E; }

// ---- mechanisms of layers that run their sublayers one after the other (ragged_mix.cu) ------------------------------------------------
// Causal depthwise convolution over time with a carried window: out[r, c] = (add_input ? in[r, c] : 0) + sum_k w[c, k] * u(r, k), where
// u(r, k) is the input taps - 1 - k tokens before row r: a row of the same entry, or the sequence's window (its last taps - 1 inputs,
// zeros for a new sequence).  The window is moved on afterwards.  single_rows: every entry brings one row (both in one launch).
struct CausalConvArgs {
    const float* in; int ld;          // [T, ld]
    int C, taps;
    const float* w;                   // [C, taps]
    float* state;                     // [slots, taps - 1, C]
    int add_input;
    ActOut out;
    int single_rows = 0;
    const float* bias = nullptr;      // nullable [C]: added to the convolution's sum
    int silu = 0;                     // 1: out = silu(sum) (after the bias)
};
int causal_conv_launch(cudaStream_t st, const RaggedBatch& rb, const CausalConvArgs& a);
int causal_conv_launch_count(const CausalConvArgs& a);

// Every entry one row: out_h = rms_in_groups(x) * norm_w, out_u = out_h + conv(out_h) over the carried window, window moved on -- one launch,
// for the sizes norm_conv_step_fits() accepts (the others take rms_rows + causal_conv)
bool norm_conv_step_fits(int W, int groups, int taps);
int norm_conv_step_launch(cudaStream_t st, const RaggedBatch& rb, const float* x, int ldx, int W, int groups, float eps, const float* norm_w,
                          int taps, const float* conv_w, float* state, const ActOut& out_h, const ActOut& out_u);

// Latent attention, first half: proj [T, ld] holds the query latent (q_rank columns) and the key / value latent (kv_rank columns).
// Each is RMS-normed with its weight; the query latent goes to cq, the key / value latent to the sequence's page at the row's position
// (one "head" of width kv_rank: the pool serves as keys and as values).
struct LatentPrepArgs {
    const float* proj; int ld;
    int q_rank, kv_rank;
    const float* q_w; const float* kv_w;
    float eps;
    ActOut cq;
    ActOut ckv;                       // optional: the normalised key / value latent of the step's rows, as an operand for further linears
    void* pool; int kv_f32; long long kv_lo_off;
    const int* block_table; int max_pages;
};
int latent_prep_launch(cudaStream_t st, const RaggedBatch& rb, const LatentPrepArgs& a);

// Block-diagonal linear: out[r, h * n_out + i] = sum_j in[r, h * n_in + j] * w[(h * n_in + j) * n_out + i], every product and sum in
// f32 in the order j = 0, 1, ...  (w is stored input-major per head: [H, n_in, n_out] bf16).
int headwise_linear_launch(cudaStream_t st, const ActOut& in, const bf16* w, int T, int H, int n_in, int n_out, const ActOut& out);

// Gated linear attention.  proj [T, ld] holds q | k | v | g | a (H*d, H*d, H*dv, H*dv, rank columns).  Per head and key channel the
// decay is sigmoid(z)^(1 / tau), z = a2 a + b (all f32); S_t = diag(decay_t) S_(t-1) + k_t v_t^T; o_t = S_t^T (q_t * q_scale); then
// out = rms_norm_over_dv(o) * norm_w * silu(g).  The state [slots, H, d, dv] is f32 and carried in place.
struct GlaArgs {
    const float* proj; int ld;
    int H, d, dv, rank;
    const float* a2;                  // [rank, H * d] f32 (the second factor of the decay's projection, transposed)
    const float* a2_b;                // [H * d]
    float inv_tau, q_scale, eps;
    const float* norm_w;              // [dv]
    float* state;
    float* decay;                     // [T, H * d] scratch
    float* y;                         // [T, H * dv] scratch
    ActOut out;                       // [T, H * dv]
    // long portions run as segments side by side (see gla_scan_kernel): scratch for their local / start states and decay products,
    // gla_seg_floats(entries, ...) floats in all; nullptr = never segment
    float* seg_state = nullptr; float* seg_decay = nullptr;
    int max_len = 0;                  // rows of the longest entry
};
int gla_mixer_launch(cudaStream_t st, const RaggedBatch& rb, const GlaArgs& a);
int gla_launch_count(bool has_seg_scratch, int max_len);
size_t gla_seg_floats(int entries, int H, int d, int dv);
size_t gla_seg_decay_offset(int entries, int H, int d, int dv);

// Selective scan with a state per channel (Mamba-1).  u [T, ldu] the convolved, activated inputs (inner columns); low [T, ldl] holds
// dt_low | B | C (dt_rank, N, N columns); z [T, ldz] the gate's pre-activations.  Per channel c and state n, all in f32:
//   dt_c = softplus(w_dt[c, :] . dt_low + dt_b[c]);  S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c u_c B_n;  y_c = sum_n S[c, n] C_n + D_c u_c
// out = y * silu(z).  The state [slots, inner, N] is carried in place.
struct Mamba1Args {
    const float* u; int ldu;
    const float* low; int ldl;
    const float* z; int ldz;
    int inner, N, dt_rank;
    const float* w_dtT;               // [dt_rank, inner] f32: the step sizes' projection, transposed
    const float* dt_b;                // [inner]
    float* dt; int lddt;              // [T, lddt] scratch: the step sizes
    const float* A;                   // [inner, N] f32, already -exp(A_log)
    const float* D;                   // [inner]
    float* state;
    ActOut out;                       // [T, inner]
    // long portions run as segments side by side (see ragged_scan.cu): scratch for their local / start states and step-size sums,
    // mamba1_seg_floats(entries, ...) floats in all; nullptr = never segment
    float* seg_state = nullptr; float* seg_dt = nullptr;
    int max_len = 0;                  // rows of the longest entry
};
int mamba1_scan_launch(cudaStream_t st, const RaggedBatch& rb, const Mamba1Args& a);
int mamba1_launch_count(bool has_seg_scratch, int max_len);
size_t mamba1_seg_floats(int entries, int inner, int N);
size_t mamba1_seg_dt_offset(int entries, int inner, int N);

// Matrix memory with exponential gates and a running maximum (mLSTM).  proj [T, ld] holds, from column col0 on,
// q | k | v | g | i | f  (H*d, H*d, H*dv, H*dv, H, H columns).  Per head, all in f32, with c = gate_cap:
//   ig = c tanh((i + i_b) / c);  fg = log sigmoid(c tanh((f + f_b) / c));  m_t = max(fg + m_(t-1), ig)
//   S_t = exp(fg + m_(t-1) - m_t) S_(t-1) + exp(ig - m_t) k v^T;  n_t likewise from k;  o = S_t^T (q * q_scale) / (max(|n_t . q q_scale|, exp(-m_t)) + 1e-6)
//   out = o / sqrt(mean_dv(o^2) + eps) * norm_w * sigmoid(g)
// State per slot: S [slots, H, d, dv], n [slots, H, d], m [slots, H] (zeros for a new sequence), carried in place.
struct MlstmArgs {
    const float* proj; int ld; int col0;
    int H, d, dv;
    float gate_cap, q_scale, eps;
    const float* i_b; const float* f_b;   // [H]
    const float* norm_w;              // [H * dv]
    float* S; float* n; float* m;
    float* y;                         // [T, H * dv] scratch: S^T q before the division
    float* gates;                     // [4, T, H] scratch: decay, input weight, exp(-m), n . q per token and head
    ActOut out;                       // [T, H * dv]
    // long portions run as segments side by side: scratch for their local / start states ([d, dv + 1] per head, the normaliser as
    // the last column) and decay products, mlstm_seg_floats(entries, ...) floats in all; nullptr = never segment
    float* seg_state = nullptr; float* seg_decay = nullptr;
    int max_len = 0;                  // rows of the longest entry
};
int mlstm_mixer_launch(cudaStream_t st, const RaggedBatch& rb, const MlstmArgs& a);
int mlstm_launch_count(bool has_seg_scratch, int max_len);
size_t mlstm_seg_floats(int entries, int H, int d, int dv);
size_t mlstm_seg_decay_offset(int entries, int H, int d, int dv);

// dst[r, c] = cap * tanh(src[r, c] / cap) for c < V (cap <= 0: a plain copy)
int softcap_rows_launch(cudaStream_t st, const float* src, int lds, int R, int V, float cap, float* dst, int ldd);

// Greedy feedback for on-device decode loops: token = argmax of logits row e (lowest index among maxima; 64 partial results per
// row in part_val / part_idx, then one block) -> ids[e], recorded at out[e * out_stride + *step]; row_pos[e] and ent_pos0[e] move on
// by one; *step is bumped once.
int greedy_advance_launch(cudaStream_t st, const float* logits, int V, int E, float* part_val, int* part_idx, int* ids, int* row_pos,
                          int* ent_pos0, uint32_t* out, int out_stride, int* step);
int gather_rows_launch(cudaStream_t st, const float* src, int lds, const int* rows, int R, int W, float* dst, int ldd);

}  // namespace cb
