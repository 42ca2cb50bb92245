// Ragged-batch kernels of layers that run their sublayers one after the other (see ragged.cuh): a carried causal convolution in
// front of a sublayer, latent attention (only a normalised low-rank row is kept
// per token; the per-head key and value maps are applied to the query and to the attention's output instead), gated linear
// attention with a decay per key channel, and a soft cap on the logits.  All of it is f32 arithmetic on CUDA cores; a row's result
// depends on its own sequence only (every sum runs in an order fixed by the row's position and the launch constants).
#include "ragged.cuh"
#include "ragged_dev.cuh"
#include "decode.cuh"

#include <algorithm>

namespace cb {

namespace {

inline int last_err() { return (int)cudaGetLastError(); }

// ---------------------------------------------------------------------------------------------------------------- convolution
__global__ void causal_conv_rows_kernel(RaggedBatch rb, CausalConvArgs a) {
    const int r = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= a.C) return;
    const int e = rb.row_entry[r], i = r - rb.ent_row0[e], slot = rb.ent_slot[e], taps = a.taps;
    const float* win = a.state + (size_t)slot * (taps - 1) * a.C;
    const float own = a.in[(size_t)r * a.ld + c];
    float acc = 0.f;
    for (int k = 0; k < taps; ++k) {
        const int back = taps - 1 - k;                   // this tap reads the input `back` tokens ago
        const float u = back == 0 ? own : (i - back >= 0) ? a.in[(size_t)(r - back) * a.ld + c] : win[(size_t)(taps - 1 + i - back) * a.C + c];
        acc = fmaf(a.w[(size_t)c * taps + k], u, acc);
    }
    if (a.bias) acc += a.bias[c];
    if (a.silu) acc = acc / (1.f + __expf(-acc));
    store_act(a.out, r, c, a.add_input ? own + acc : acc);
}
// New window = the last taps - 1 inputs of the sequence (older ones shift down when the entry is shorter than the window).
__global__ void causal_conv_window_kernel(RaggedBatch rb, CausalConvArgs a) {
    const int e = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= a.C) return;
    const int len = rb.ent_len[e], r0 = rb.ent_row0[e], slot = rb.ent_slot[e], nwin = a.taps - 1;
    float* win = a.state + (size_t)slot * nwin * a.C;
    for (int i = 0; i < nwin; ++i) {
        const int src = len - nwin + i;                  // index among this entry's rows
        win[(size_t)i * a.C + c] = (src >= 0) ? a.in[(size_t)(r0 + src) * a.ld + c] : win[(size_t)(i + len) * a.C + c];
    }
}
// Every entry one token: the convolution and the window shift in one pass; thread = (entry, channel) owns its window column.
__global__ void causal_conv_step_kernel(RaggedBatch rb, CausalConvArgs a) {
    const int e = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= a.C) return;
    const int r = rb.ent_row0[e], slot = rb.ent_slot[e], taps = a.taps;
    float* win = a.state + (size_t)slot * (taps - 1) * a.C;
    const float u = a.in[(size_t)r * a.ld + c];
    float acc = 0.f;
    for (int k = 0; k < taps - 1; ++k) {
        const float w = win[(size_t)k * a.C + c];
        acc = fmaf(a.w[(size_t)c * taps + k], w, acc);
        if (k > 0) win[(size_t)(k - 1) * a.C + c] = w;
    }
    acc = fmaf(a.w[(size_t)c * taps + taps - 1], u, acc);
    if (taps > 1) win[(size_t)(taps - 2) * a.C + c] = u;
    if (a.bias) acc += a.bias[c];
    if (a.silu) acc = acc / (1.f + __expf(-acc));
    store_act(a.out, r, c, a.add_input ? u + acc : acc);
}

__global__ void softcap_rows_kernel(const float* __restrict__ src, int lds, int V, float cap, float* __restrict__ dst, int ldd) {
    const int r = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= V) return;
    const float z = src[(size_t)r * lds + c];
    dst[(size_t)r * ldd + c] = cap > 0.f ? cap * tanhf(z / cap) : z;
}

// ---------------------------------------------------------------------------------------------------------------- latent attention
// Block per row: the two latents one after the other, each with its own sum of squares (thread-strided partial sums, then a fixed
// tree), the second stored into the sequence's page.
template <typename KT>
__global__ void __launch_bounds__(256) latent_prep_kernel(RaggedBatch rb, LatentPrepArgs a) {
    __shared__ float red[8];
    const int r = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int e = rb.row_entry[r], pos = rb.row_pos[r], slot = rb.ent_slot[e];
    const int page = a.block_table[(size_t)slot * a.max_pages + pos / KV_PAGE];
    KT* dst = (KT*)a.pool + ((size_t)page * KV_PAGE + (pos % KV_PAGE)) * a.kv_rank;
    for (int seg = 0; seg < 2; ++seg) {
        const int n = seg ? a.kv_rank : a.q_rank;
        const float* src = a.proj + (size_t)r * a.ld + (seg ? a.q_rank : 0);
        const float* w = seg ? a.kv_w : a.q_w;
        float ss = 0.f;
        for (int c = threadIdx.x; c < n; c += 256) ss = fmaf(src[c], src[c], ss);
        ss = warp_sum(ss);
        if (seg) __syncthreads();
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) tot += red[k];
        const float inv = 1.f / sqrtf(tot / (float)n + a.eps);
        for (int c = threadIdx.x; c < n; c += 256) {
            const float v = src[c] * inv * w[c];
            if (seg) { kv_store<KT>(dst + c, v, a.kv_lo_off); if (a.ckv.f || a.ckv.hi) store_act(a.ckv, r, c, v); }
            else store_act(a.cq, r, c, v);
        }
    }
}

// Block = (HW_ROWS rows, head): the rows' input slices sit in shared memory, a thread owns output columns i, i + 128, ... and walks the
// head's [n_in, n_out] matrix down its column (neighbouring threads read neighbouring weights).
constexpr int HW_ROWS = 8;
__device__ __forceinline__ float act_load(const ActOut& o, int r, int c) {
    if (o.f) return o.f[(size_t)r * o.ldf + c];
    const bf16* p = o.hi + (size_t)r * o.ldb + c;
    return __bfloat162float(*p) + (o.lo_off ? __bfloat162float(p[o.lo_off]) : 0.f);
}
__global__ void __launch_bounds__(128) headwise_linear_kernel(ActOut in, const bf16* __restrict__ w, int T, int n_in, int n_out, ActOut out) {
    extern __shared__ float hw_in[];                      // [HW_ROWS][n_in]
    const int r0 = blockIdx.x * HW_ROWS, h = blockIdx.y, nr = min(HW_ROWS, T - r0);
    for (int i = threadIdx.x; i < HW_ROWS * n_in; i += blockDim.x) {
        const int rr = i / n_in, j = i - rr * n_in;
        hw_in[i] = rr < nr ? act_load(in, r0 + rr, h * n_in + j) : 0.f;
    }
    __syncthreads();
    const bf16* wh = w + (size_t)h * n_in * n_out;
    for (int i = threadIdx.x; i < n_out; i += blockDim.x) {
        float acc[HW_ROWS];
#pragma unroll
        for (int rr = 0; rr < HW_ROWS; ++rr) acc[rr] = 0.f;
        for (int j = 0; j < n_in; ++j) {
            const float wv = __bfloat162float(wh[(size_t)j * n_out + i]);
#pragma unroll
            for (int rr = 0; rr < HW_ROWS; ++rr) acc[rr] = fmaf(hw_in[rr * n_in + j], wv, acc[rr]);
        }
#pragma unroll
        for (int rr = 0; rr < HW_ROWS; ++rr) if (rr < nr) store_act(out, r0 + rr, h * n_out + i, acc[rr]);
    }
}

// Up to HWF_ROWS rows (a decode step): block = (128 output columns, head); its sixteen warps split the head's n_in input rows between
// them, a lane owns four neighbouring columns (one 8-byte load of the bf16 weights per input row, the warp reads 256 contiguous bytes;
// a warp's handful of rows are all requested before the first is used), and the warps' partial sums meet in warp order.
constexpr int HWF_ROWS = 4, HWF_WARPS = 16, HWF_COLS = 128;
__global__ void __launch_bounds__(HWF_WARPS * 32) headwise_few_kernel(ActOut in, const bf16* __restrict__ w, int T, int n_in, int n_out, ActOut out) {
    extern __shared__ float hwf_s[];                      // [T][n_in] inputs, then [warps][HWF_ROWS][HWF_COLS] partial sums
    float* xin = hwf_s;
    float* part = hwf_s + (((size_t)T * n_in + 3) & ~(size_t)3);
    const int h = blockIdx.y, c0 = blockIdx.x * HWF_COLS, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < T * n_in; i += blockDim.x) { const int rr = i / n_in, j = i - rr * n_in; xin[i] = act_load(in, rr, h * n_in + j); }
    __syncthreads();
    const int col = c0 + 4 * lane, per = (n_in + HWF_WARPS - 1) / HWF_WARPS, j0 = warp * per, j1 = min(n_in, j0 + per);
    const bool vec = (n_out & 3) == 0;                     // (then every group of four starts on an 8-byte boundary)
    float acc[HWF_ROWS][4] = {};
    const bf16* wh = w + (size_t)h * n_in * n_out + col;
    for (int jb = j0; jb < j1; jb += 8) {
        float wv[8][4];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int j = jb + u;
            wv[u][0] = wv[u][1] = wv[u][2] = wv[u][3] = 0.f;
            if (j < j1 && col < n_out) {
                if (vec) { const uint2 t = *reinterpret_cast<const uint2*>(wh + (size_t)j * n_out); wv[u][0] = bf16lo(t.x); wv[u][1] = bf16hi(t.x); wv[u][2] = bf16lo(t.y); wv[u][3] = bf16hi(t.y); }
                else for (int c = 0; c < 4; ++c) if (col + c < n_out) wv[u][c] = __bfloat162float(wh[(size_t)j * n_out + c]);
            }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int j = jb + u;
            if (j >= j1) break;
#pragma unroll
            for (int rr = 0; rr < HWF_ROWS; ++rr)
                if (rr < T) {
                    const float xv = xin[rr * n_in + j];
#pragma unroll
                    for (int c = 0; c < 4; ++c) acc[rr][c] = fmaf(xv, wv[u][c], acc[rr][c]);
                }
        }
    }
#pragma unroll
    for (int rr = 0; rr < HWF_ROWS; ++rr)
        *reinterpret_cast<float4*>(part + ((size_t)warp * HWF_ROWS + rr) * HWF_COLS + 4 * lane) = make_float4(acc[rr][0], acc[rr][1], acc[rr][2], acc[rr][3]);
    __syncthreads();
    for (int i = threadIdx.x; i < T * HWF_COLS; i += blockDim.x) {
        const int rr = i / HWF_COLS, c = i - rr * HWF_COLS;
        if (c0 + c >= n_out) continue;
        float sum = 0.f;
#pragma unroll
        for (int wq = 0; wq < HWF_WARPS; ++wq) sum += part[((size_t)wq * HWF_ROWS + rr) * HWF_COLS + c];
        store_act(out, rr, h * n_out + c0 + c, sum);
    }
}

// Every entry one token: the sublayer's norm (RMS in equal groups), the convolution over the carried window and the window's shift
// in one pass.  Block per entry, NCS columns per thread; everything the row needs (its x, the norm and tap weights, the window) is
// requested up front, so the kernel costs one trip to memory.  h = norm output goes to out_h, h + conv(h) to out_u.
constexpr int NCS_COLS = 4, NCS_GROUPS = 8;
template <int TAPS>
__global__ void __launch_bounds__(1024) norm_conv_step_kernel(RaggedBatch rb, const float* __restrict__ x, int ldx, int W, int groups, float eps,
                                                              const float* __restrict__ nw, const float* __restrict__ cw, float* state,
                                                              ActOut out_h, ActOut out_u) {
    __shared__ float red[NCS_GROUPS][32];
    const int e = blockIdx.x, r = rb.ent_row0[e], slot = rb.ent_slot[e], lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    const float* xr = x + (size_t)r * ldx;
    float* win = state + (size_t)slot * (TAPS - 1) * W;
    const int part = W / groups;
    float xv[NCS_COLS], wn[NCS_COLS], tw[NCS_COLS][TAPS], old[NCS_COLS][TAPS > 1 ? TAPS - 1 : 1];
#pragma unroll
    for (int k = 0; k < NCS_COLS; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        const bool in = c < W;
        xv[k] = in ? xr[c] : 0.f;
        wn[k] = in ? nw[c] : 0.f;
#pragma unroll
        for (int t = 0; t < TAPS; ++t) tw[k][t] = in ? cw[(size_t)c * TAPS + t] : 0.f;
#pragma unroll
        for (int t = 0; t < TAPS - 1; ++t) old[k][t] = in ? win[(size_t)t * W + c] : 0.f;
    }
    for (int g = 0; g < groups; ++g) {                      // a group's sum of squares: a thread's own columns in order, the warp's tree, the warps in order
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < NCS_COLS; ++k) { const int c = threadIdx.x + k * blockDim.x; if (c < W && c / part == g) ss = fmaf(xv[k], xv[k], ss); }
        ss = warp_sum(ss);
        if (lane == 0) red[g][warp] = ss;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < NCS_COLS; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (c >= W) continue;
        const int g = c / part;
        float tot = 0.f;
        for (int wq = 0; wq < nwarp; ++wq) tot += red[g][wq];
        const float u = xv[k] * (1.f / sqrtf(tot / (float)part + eps)) * wn[k];
        float acc = 0.f;
#pragma unroll
        for (int t = 0; t < TAPS - 1; ++t) {
            acc = fmaf(tw[k][t], old[k][t], acc);
            if (t > 0) win[(size_t)(t - 1) * W + c] = old[k][t];
        }
        acc = fmaf(tw[k][TAPS - 1], u, acc);
        if (TAPS > 1) win[(size_t)(TAPS - 2) * W + c] = u;
        store_act(out_h, r, c, u);
        store_act(out_u, r, c, u + acc);
    }
}

// ---------------------------------------------------------------------------------------------------------------- gated linear attention
// decay[r, c] = sigmoid(z)^(1 / tau) = exp(log_sigmoid(z) / tau), z = a2[c, :] . a[r, :] + b[c]; log_sigmoid(z) = min(z, 0) - log1p(e^-|z|)
// (a2 is stored transposed, [rank, H * d]: neighbouring threads read neighbouring channels; GLA_DROWS rows share each weight)
constexpr int GLA_DROWS = 8;
__global__ void __launch_bounds__(128) gla_decay_kernel(GlaArgs a, int T) {
    extern __shared__ float lowrank[];                    // [GLA_DROWS][rank]
    const int r0 = blockIdx.x * GLA_DROWS, C = a.H * a.d, nr = min(GLA_DROWS, T - r0);
    for (int i = threadIdx.x; i < GLA_DROWS * a.rank; i += blockDim.x) {
        const int rr = i / a.rank, j = i - rr * a.rank;
        lowrank[i] = rr < nr ? a.proj[(size_t)(r0 + rr) * a.ld + 2 * C + 2 * a.H * a.dv + j] : 0.f;
    }
    __syncthreads();
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        float z[GLA_DROWS];
        const float b = a.a2_b[c];
#pragma unroll
        for (int rr = 0; rr < GLA_DROWS; ++rr) z[rr] = b;
#pragma unroll 8
        for (int j = 0; j < a.rank; ++j) {
            const float wv = a.a2[(size_t)j * C + c];
#pragma unroll
            for (int rr = 0; rr < GLA_DROWS; ++rr) z[rr] = fmaf(wv, lowrank[rr * a.rank + j], z[rr]);
        }
#pragma unroll
        for (int rr = 0; rr < GLA_DROWS; ++rr)
            if (rr < nr) a.decay[(size_t)(r0 + rr) * C + c] = expf((fminf(z[rr], 0.f) - log1pf(expf(-fabsf(z[rr])))) * a.inv_tau);
    }
}

// The recurrence.  Block = (entry, head, slice of GLA_COLS value columns); thread (p, ns) keeps state rows ns * R .. ns * R + R - 1 of
// column p in registers for the whole portion.  One token costs one multiply-add per state element and another for the output, so
// what would serialise the loop is fetching its operands: the step inputs (v slice, k, q, decay) of GLA_CH tokens at a time are
// staged in shared memory with cp.async, double-buffered.  Every R-run of a staged vector is followed by 4 pad floats, which
// spreads the eight runs a warp reads at once over all banks; rows past d stay zero from the start and leave the state at zero.
constexpr int GLA_NS = 8, GLA_COLS = 16, GLA_CH = 16;
__host__ __device__ inline int gla_idx(int n, int R) { return n + 4 * (n / R); }
__host__ __device__ inline int gla_npad(int R) { return 8 * (R + 4); }
// Long portions are cut into GLA_SEGS segments that run side by side (one resident warp per scheduler waits on its own dependent
// chain most of the time): the recurrence is linear with a decay per state ROW, so
//   S_end(segment) = diag(product of the segment's decays) * S_start + S_local(segment run from zero).
// MODE 1 runs every segment from zero and leaves S_local and the decay products; gla_seg_prefix_kernel turns them into each segment's
// start state (and the sequence's new state); MODE 2 is the scan proper from those start states.  MODE 0 = one segment, everything.
constexpr int GLA_SEGS = 4, GLA_SEG_MIN = 512;
__host__ __device__ inline int gla_seg_len(int len) { return ((len + GLA_SEGS - 1) / GLA_SEGS + GLA_CH - 1) / GLA_CH * GLA_CH; }
template <int R, int MODE>
__global__ void __launch_bounds__(GLA_COLS * GLA_NS) gla_scan_kernel(RaggedBatch rb, GlaArgs a) {
    extern __shared__ __align__(16) float gla_s[];
    const int e = MODE == 0 ? blockIdx.x : blockIdx.x / GLA_SEGS, seg = MODE == 0 ? 0 : blockIdx.x % GLA_SEGS;
    const int h = blockIdx.y, ns = threadIdx.x & (GLA_NS - 1), pl = threadIdx.x / GLA_NS;
    const int p0 = blockIdx.z * GLA_COLS, p = p0 + pl;
    const int d = a.d, dv = a.dv, C = a.H * d;
    const bool live = p < dv;
    const int full_len = rb.ent_len[e], slot = rb.ent_slot[e];
    const int seg_len = MODE == 0 ? full_len : gla_seg_len(full_len), seg0 = seg * seg_len;
    if (seg0 >= full_len) return;                             // (a short entry has fewer segments)
    const int len = min(seg_len, full_len - seg0), r0 = rb.ent_row0[e] + seg0;
    const int ncol = min(GLA_COLS, dv - p0);
    const int NP = gla_npad(R), per_tok = GLA_COLS + 3 * NP;
    float* stage[2] = {gla_s, gla_s + GLA_CH * per_tok};
    float* S = MODE == 0 ? a.state + (((size_t)slot * a.H + h) * d) * dv : a.seg_state + ((((size_t)e * GLA_SEGS + seg) * a.H + h) * d) * dv;
    const int n0 = ns * R;
    for (int i = threadIdx.x; i < 2 * GLA_CH * per_tok; i += blockDim.x) gla_s[i] = 0.f;
    __syncthreads();
    float s[R], dprod[MODE == 1 ? R : 1];
#pragma unroll
    for (int i = 0; i < R; ++i) s[i] = (MODE != 1 && n0 + i < d && live) ? S[(size_t)(n0 + i) * dv + p] : 0.f;
    if constexpr (MODE == 1) {
#pragma unroll
        for (int i = 0; i < R; ++i) dprod[i] = 1.f;
    }
    const int qoff = h * d, koff = C + h * d, voff = 2 * C + h * dv + p0;
    // 16-byte copies when every piece starts on a 16-byte boundary (the usual geometry), 4-byte copies otherwise
    const bool wide = ((d | dv | a.ld | C) & 3) == 0 && (R & 3) == 0;
    auto fetch = [&](int c, float* dst) {                     // tokens [c * GLA_CH, ...) of the portion
        const int t0 = c * GLA_CH, nt = min(GLA_CH, len - t0);
        if (wide) {                                           // 8 threads per token: v (4 pieces), then k, q, decay (d / 4 pieces each)
            const int t = threadIdx.x >> 3, q = threadIdx.x & 7, nq = d >> 2;
            if (t < nt) {
                const float* row = a.proj + (size_t)(r0 + t0 + t) * a.ld;
                const float* dec = a.decay + (size_t)(r0 + t0 + t) * C + h * d;
                float* d0 = dst + t * per_tok;
                for (int k = q; k < GLA_COLS / 4 + 3 * nq; k += 8) {
                    if (k < GLA_COLS / 4) { if (4 * k < ncol) cp_async16s(d0 + 4 * k, row + voff + 4 * k); }
                    else {
                        const int which = (k - GLA_COLS / 4) / nq, n = 4 * ((k - GLA_COLS / 4) % nq);
                        const float* src = which == 0 ? row + koff + n : which == 1 ? row + qoff + n : dec + n;
                        cp_async16s(d0 + GLA_COLS + which * NP + gla_idx(n, R), src);
                    }
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            return;
        }
        const int src_tok = GLA_COLS + 3 * d;
        for (int i = threadIdx.x; i < nt * src_tok; i += blockDim.x) {
            const int t = i / src_tok, j = i - t * src_tok, r = r0 + t0 + t;
            const float* row = a.proj + (size_t)r * a.ld;
            const float* src;
            int o;
            if (j < GLA_COLS) { if (j >= ncol) continue; src = row + voff + j; o = j; }
            else {
                const int which = (j - GLA_COLS) / d, n = (j - GLA_COLS) % d;
                src = which == 0 ? row + koff + n : which == 1 ? row + qoff + n : a.decay + (size_t)r * C + h * d + n;
                o = GLA_COLS + which * NP + gla_idx(n, R);
            }
            cp_async4(dst + t * per_tok + o, src);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const int nch = (len + GLA_CH - 1) / GLA_CH;
    fetch(0, stage[0]);
    for (int c = 0; c < nch; ++c) {
        if (c + 1 < nch) { fetch(c + 1, stage[(c + 1) & 1]); asm volatile("cp.async.wait_group 1;" ::: "memory"); }
        else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        const float* st = stage[c & 1];
        const int nt = min(GLA_CH, len - c * GLA_CH);
        for (int t = 0; t < nt; ++t) {
            const float* tk = st + t * per_tok;
            const float xv = live ? tk[pl] : 0.f;
            const float* kp = tk + GLA_COLS + gla_idx(n0, R);
            float y0 = 0.f, y1 = 0.f;
            if ((R & 3) == 0) {
                const float4* K4 = reinterpret_cast<const float4*>(kp);
                const float4* Q4 = reinterpret_cast<const float4*>(kp + NP);
                const float4* A4 = reinterpret_cast<const float4*>(kp + 2 * NP);
                if constexpr (MODE == 1) {                    // state and decay products only
#pragma unroll
                    for (int i = 0; i < R / 4; ++i) {
                        const float4 k = K4[i], al = A4[i];
                        s[4 * i]     = fmaf(al.x, s[4 * i],     k.x * xv); s[4 * i + 1] = fmaf(al.y, s[4 * i + 1], k.y * xv);
                        s[4 * i + 2] = fmaf(al.z, s[4 * i + 2], k.z * xv); s[4 * i + 3] = fmaf(al.w, s[4 * i + 3], k.w * xv);
                        dprod[4 * i] *= al.x; dprod[4 * i + 1] *= al.y; dprod[4 * i + 2] *= al.z; dprod[4 * i + 3] *= al.w;
                    }
                    continue;
                }
#pragma unroll
                for (int i = 0; i < R / 4; ++i) {
                    const float4 k = K4[i], q = Q4[i], al = A4[i];
                    s[4 * i]     = fmaf(al.x, s[4 * i],     k.x * xv); y0 = fmaf(s[4 * i],     q.x, y0);
                    s[4 * i + 1] = fmaf(al.y, s[4 * i + 1], k.y * xv); y1 = fmaf(s[4 * i + 1], q.y, y1);
                    s[4 * i + 2] = fmaf(al.z, s[4 * i + 2], k.z * xv); y0 = fmaf(s[4 * i + 2], q.z, y0);
                    s[4 * i + 3] = fmaf(al.w, s[4 * i + 3], k.w * xv); y1 = fmaf(s[4 * i + 3], q.w, y1);
                }
            }
            float y = y0 + y1;
#pragma unroll
            for (int o = GLA_NS / 2; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
            if (ns == 0 && live) a.y[(size_t)(r0 + c * GLA_CH + t) * a.H * dv + h * dv + p] = y * a.q_scale;
        }
        __syncthreads();                                      // the stage is free for chunk c + 2
    }
    if (MODE == 2) return;                                    // the prefix kernel already wrote the sequence's new state
#pragma unroll
    for (int i = 0; i < R; ++i) if (n0 + i < d && live) S[(size_t)(n0 + i) * dv + p] = s[i];
    if constexpr (MODE == 1) {
        if (pl == 0 && blockIdx.z == 0) {
#pragma unroll
            for (int i = 0; i < R; ++i) if (n0 + i < d) a.seg_decay[(((size_t)e * GLA_SEGS + seg) * a.H + h) * d + n0 + i] = dprod[i];
        }
    }
}
// Start state of every segment, in order: seg_state[k] holds S_local on entry and S_start(k) on exit; the slot gets the end state.
__global__ void gla_seg_prefix_kernel(RaggedBatch rb, GlaArgs a) {
    const int e = blockIdx.x, h = blockIdx.y, np = a.d * a.dv;
    const int len = rb.ent_len[e], slot = rb.ent_slot[e], nseg = (len + gla_seg_len(len) - 1) / gla_seg_len(len);
    float* S = a.state + ((size_t)slot * a.H + h) * np;
    for (int i = blockIdx.z * blockDim.x + threadIdx.x; i < np; i += gridDim.z * blockDim.x) {
        const int n = i / a.dv;
        float cur = S[i];
        for (int k = 0; k < nseg; ++k) {
            float* loc = a.seg_state + (((size_t)e * GLA_SEGS + k) * a.H + h) * np + i;
            const float l = *loc;
            *loc = cur;
            cur = fmaf(a.seg_decay[(((size_t)e * GLA_SEGS + k) * a.H + h) * a.d + n], cur, l);
        }
        S[i] = cur;
    }
}

// out[r, h * dv + c] = y / sqrt(mean_c(y^2) + eps) * w[c] * silu(g[r, h * dv + c]): one warp per (row, head)
__global__ void __launch_bounds__(128) gla_out_kernel(GlaArgs a, int T) {
    const int r = blockIdx.x, h = blockIdx.y * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (h >= a.H) return;
    const int dv = a.dv;
    const float* y = a.y + (size_t)r * a.H * dv + h * dv;
    const float* g = a.proj + (size_t)r * a.ld + 2 * a.H * a.d + a.H * dv + h * dv;
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) ss = fmaf(y[c], y[c], ss);
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / (float)dv + a.eps);
    for (int c = lane; c < dv; c += 32) store_act(a.out, r, h * dv + c, y[c] * inv * a.norm_w[c] * silu_f(g[c]));
}

}  // namespace

// ---------------------------------------------------------------------------------------------------------------- launchers
int causal_conv_launch_count(const CausalConvArgs& a) { return (a.single_rows || a.taps <= 1) ? 1 : 2; }
int causal_conv_launch(cudaStream_t st, const RaggedBatch& rb, const CausalConvArgs& a) {
    if (a.taps < 1 || a.C < 1 || !a.in) return -1000;
    const dim3 grid((a.C + 127) / 128, a.single_rows ? rb.E : rb.T);
    if (a.single_rows) {
        causal_conv_step_kernel<<<grid, 128, 0, st>>>(rb, a);
        return last_err();
    }
    causal_conv_rows_kernel<<<grid, 128, 0, st>>>(rb, a);
    if (const int e = last_err()) return e;
    if (a.taps > 1) causal_conv_window_kernel<<<dim3((a.C + 127) / 128, rb.E), 128, 0, st>>>(rb, a);
    return last_err();
}
bool norm_conv_step_fits(int W, int groups, int taps) { return groups >= 1 && groups <= NCS_GROUPS && W % groups == 0 && taps >= 1 && taps <= 4 && W <= 1024 * NCS_COLS; }
int norm_conv_step_launch(cudaStream_t st, const RaggedBatch& rb, const float* x, int ldx, int W, int groups, float eps, const float* norm_w,
                          int taps, const float* conv_w, float* state, const ActOut& out_h, const ActOut& out_u) {
    if (!norm_conv_step_fits(W, groups, taps)) return -1000;
    const int threads = std::min(1024, std::max(128, ((W + NCS_COLS - 1) / NCS_COLS + 31) / 32 * 32));
    switch (taps) {
        case 1: norm_conv_step_kernel<1><<<rb.E, threads, 0, st>>>(rb, x, ldx, W, groups, eps, norm_w, conv_w, state, out_h, out_u); break;
        case 2: norm_conv_step_kernel<2><<<rb.E, threads, 0, st>>>(rb, x, ldx, W, groups, eps, norm_w, conv_w, state, out_h, out_u); break;
        case 3: norm_conv_step_kernel<3><<<rb.E, threads, 0, st>>>(rb, x, ldx, W, groups, eps, norm_w, conv_w, state, out_h, out_u); break;
        default: norm_conv_step_kernel<4><<<rb.E, threads, 0, st>>>(rb, x, ldx, W, groups, eps, norm_w, conv_w, state, out_h, out_u); break;
    }
    return last_err();
}
int softcap_rows_launch(cudaStream_t st, const float* src, int lds, int R, int V, float cap, float* dst, int ldd) {
    softcap_rows_kernel<<<dim3((V + 255) / 256, R), 256, 0, st>>>(src, lds, V, cap, dst, ldd);
    return last_err();
}
int latent_prep_launch(cudaStream_t st, const RaggedBatch& rb, const LatentPrepArgs& a) {
    if (a.q_rank < 1 || a.kv_rank < 1) return -1000;
    if (a.kv_f32) latent_prep_kernel<float><<<rb.T, 256, 0, st>>>(rb, a);
    else latent_prep_kernel<bf16><<<rb.T, 256, 0, st>>>(rb, a);
    return last_err();
}
int headwise_linear_launch(cudaStream_t st, const ActOut& in, const bf16* w, int T, int H, int n_in, int n_out, const ActOut& out) {
    const size_t smem = (size_t)HW_ROWS * n_in * sizeof(float);
    if ((!in.f && !in.hi) || smem > 200 * 1024) return -1000;
    if (T <= HWF_ROWS) {
        const size_t sf = ((size_t)((T * n_in + 3) & ~3) + (size_t)HWF_WARPS * HWF_ROWS * HWF_COLS) * sizeof(float);
        static SmemOptIn seen_few;
        if (const int e = ensure_dyn_smem(headwise_few_kernel, sf, seen_few)) return e;
        headwise_few_kernel<<<dim3((n_out + HWF_COLS - 1) / HWF_COLS, H), HWF_WARPS * 32, sf, st>>>(in, w, T, n_in, n_out, out);
        return last_err();
    }
    static SmemOptIn seen;
    if (const int e = ensure_dyn_smem(headwise_linear_kernel, smem, seen)) return e;
    headwise_linear_kernel<<<dim3((T + HW_ROWS - 1) / HW_ROWS, H), 128, smem, st>>>(in, w, T, n_in, n_out, out);
    return last_err();
}
int gla_launch_count(bool has_seg_scratch, int max_len) { return has_seg_scratch && max_len >= GLA_SEG_MIN ? 5 : 3; }
size_t gla_seg_floats(int entries, int H, int d, int dv) { return (size_t)entries * GLA_SEGS * H * ((size_t)d * dv + d); }
size_t gla_seg_decay_offset(int entries, int H, int d, int dv) { return (size_t)entries * GLA_SEGS * H * (size_t)d * dv; }
int gla_mixer_launch(cudaStream_t st, const RaggedBatch& rb, const GlaArgs& a) {
    if (a.d < 1 || a.d > 256 || a.dv < 1 || a.rank < 1 || a.rank > 8192) return -1000;
    const int row_blocks = (rb.T + GLA_DROWS - 1) / GLA_DROWS;      // few rows: the channels spread over blocks as well
    gla_decay_kernel<<<dim3(row_blocks, row_blocks >= 64 ? 1 : std::max(1, std::min(16, (a.H * a.d + 127) / 128))), 128, (size_t)GLA_DROWS * a.rank * sizeof(float), st>>>(a, rb.T);
    int e = last_err();
    if (e) return e;
    const int nr = (a.d + GLA_NS - 1) / GLA_NS, R = nr <= 4 ? 4 : nr <= 8 ? 8 : nr <= 16 ? 16 : 32;
    const size_t smem = (size_t)2 * GLA_CH * (GLA_COLS + 3 * gla_npad(R)) * sizeof(float);      // <= 113 KB at d = 256
    const dim3 grid(rb.E, a.H, (a.dv + GLA_COLS - 1) / GLA_COLS);
    auto run = [&](auto kern, SmemOptIn& seen, dim3 g) -> int {
        if (const int er = ensure_dyn_smem(kern, smem, seen)) return er;
        kern<<<g, GLA_COLS * GLA_NS, smem, st>>>(rb, a);
        return last_err();
    };
    auto scan = [&](auto k4, auto k8, auto k16, auto k32, SmemOptIn* seen, dim3 g) -> int {
        return R == 4 ? run(k4, seen[0], g) : R == 8 ? run(k8, seen[1], g) : R == 16 ? run(k16, seen[2], g) : run(k32, seen[3], g);
    };
    static SmemOptIn seen0[4], seen1[4], seen2[4];
    if (gla_launch_count(a.seg_state != nullptr, a.max_len) == 3) {
        e = scan(gla_scan_kernel<4, 0>, gla_scan_kernel<8, 0>, gla_scan_kernel<16, 0>, gla_scan_kernel<32, 0>, seen0, grid);
    } else {
        const dim3 ggrid(rb.E * GLA_SEGS, a.H, grid.z);
        if ((e = scan(gla_scan_kernel<4, 1>, gla_scan_kernel<8, 1>, gla_scan_kernel<16, 1>, gla_scan_kernel<32, 1>, seen1, ggrid))) return e;
        gla_seg_prefix_kernel<<<dim3(rb.E, a.H, 8), 256, 0, st>>>(rb, a);
        if ((e = last_err())) return e;
        e = scan(gla_scan_kernel<4, 2>, gla_scan_kernel<8, 2>, gla_scan_kernel<16, 2>, gla_scan_kernel<32, 2>, seen2, ggrid);
    }
    if (e) return e;
    gla_out_kernel<<<dim3(rb.T, (a.H + 3) / 4), 128, 0, st>>>(a, rb.T);
    return last_err();
}

}  // namespace cb
