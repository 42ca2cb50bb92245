// Ragged-batch kernels (see ragged.cuh).  Everything here is f32 arithmetic on CUDA cores: norms, softmax, routers, the
// recurrent state and all that enters the recurrence are kept in 32-bit; the big linears run on the tensor cores (gemm.cu) from
// the bf16 planes these kernels emit, or through linear_f32_kernel in the exact mode.
//
// A row's result depends on that row's sequence only: every reduction runs in an order fixed by the row's own position and the
// launch constants, never by what else shares the step.
#include "ragged.cuh"
#include "ragged_dev.cuh"
#include "decode.cuh"

#include <algorithm>

namespace cb {

namespace {

// ---------------------------------------------------------------------------------------------------------------- rows
__global__ void embed_scale_rows_kernel(const int* __restrict__ ids, int T, const bf16* __restrict__ embed, int W, float scale,
                                        float* __restrict__ x, int ldx) {
    const int r = blockIdx.x;
    const bf16* e = embed + (size_t)ids[r] * W;
    for (int c = threadIdx.x; c < W; c += blockDim.x) x[(size_t)r * ldx + c] = __bfloat162float(e[c]) * scale;
}

__global__ void embed_sinpos_rows_kernel(const int* __restrict__ ids, const int* __restrict__ row_pos, const bf16* __restrict__ embed, int W,
                                         const float* __restrict__ freq, float* __restrict__ x, int ldx) {
    const int r = blockIdx.x;
    const bf16* e = embed + (size_t)ids[r] * W;
    const float pos = (float)row_pos[r];
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float ang = pos * freq[c >> 1];
        x[(size_t)r * ldx + c] = __bfloat162float(e[c]) + ((c & 1) ? cosf(ang) : sinf(ang));
    }
}

// Block per row.  One input: x += rms(y1 + b1) * norm_w.  Two inputs: v = (rms(y1 + b1) * w1 + rms(y2) * w2) / 2, x += rms(v) * norm_w.
__global__ void __launch_bounds__(256) post_norm_add_kernel(const float* __restrict__ y1, int ld1, const float* __restrict__ b1, const float* __restrict__ w1,
                                                            const float* __restrict__ y2, int ld2, const float* __restrict__ w2,
                                                            const float* __restrict__ norm_w, float eps, float* __restrict__ x, int ldx, int W, ActOut planes) {
    __shared__ float red[3][8];
    const int r = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float* a = y1 + (size_t)r * ld1;
    const float* b = y2 ? y2 + (size_t)r * ld2 : nullptr;
    float* xr = x + (size_t)r * ldx;
    auto total = [&](float v, int k) {      // fixed order: thread-strided partial sums, warp tree, warps in order
        v = warp_sum(v);
        if (lane == 0) red[k][warp] = v;
        __syncthreads();
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) t += red[k][w];
        return t;
    };
    float sa = 0.f, sb = 0.f;
    for (int c = threadIdx.x; c < W; c += 256) {
        const float u = a[c] + (b1 ? b1[c] : 0.f);
        sa = fmaf(u, u, sa);
        if (b) sb = fmaf(b[c], b[c], sb);
    }
    const float ia = 1.f / sqrtf(total(sa, 0) / (float)W + eps);
    if (!b) {
        for (int c = threadIdx.x; c < W; c += 256) {
            const float nx = xr[c] + (a[c] + (b1 ? b1[c] : 0.f)) * ia * norm_w[c];
            xr[c] = nx;
            store_act(planes, r, c, nx);
        }
        return;
    }
    const float ib = 1.f / sqrtf(total(sb, 1) / (float)W + eps);
    float sv = 0.f;
    for (int c = threadIdx.x; c < W; c += 256) {
        const float v = 0.5f * ((a[c] + (b1 ? b1[c] : 0.f)) * ia * (w1 ? w1[c] : 1.f) + b[c] * ib * (w2 ? w2[c] : 1.f));
        sv = fmaf(v, v, sv);
    }
    const float iv = 1.f / sqrtf(total(sv, 2) / (float)W + eps);
    for (int c = threadIdx.x; c < W; c += 256) {
        const float v = 0.5f * ((a[c] + (b1 ? b1[c] : 0.f)) * ia * (w1 ? w1[c] : 1.f) + b[c] * ib * (w2 ? w2[c] : 1.f));
        const float nx = xr[c] + v * iv * norm_w[c];
        xr[c] = nx;
        store_act(planes, r, c, nx);
    }
}

__global__ void dyt_rows_kernel(const float* __restrict__ x, int ldx, const int* __restrict__ rows, int W, const float* __restrict__ alpha,
                                const float* __restrict__ w, const float* __restrict__ b, ActOut out) {
    const int r = blockIdx.x, src = rows ? rows[r] : r;
    const float a = *alpha;
    for (int c = threadIdx.x; c < W; c += blockDim.x) store_act(out, r, c, tanhf(a * x[(size_t)src * ldx + c]) * w[c] + b[c]);
}

// RMS norm of a row with up to two weight vectors on the one statistic.  The sum of squares runs in a fixed order (thread-strided
// partial sums, then a tree over the block), so a row's result does not depend on what else is in the step.  groups > 1: the row
// is cut into that many equal consecutive parts and each part is divided by its own root mean square.
__global__ void __launch_bounds__(256) rms_rows_kernel(const float* __restrict__ x, int ldx, const int* __restrict__ rows, int W, float eps,
                                                       const float* __restrict__ w1, ActOut out1, const float* __restrict__ w2, ActOut out2, int groups) {
    __shared__ float red[8];
    const int r = blockIdx.x, src = rows ? rows[r] : r, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float* xr = x + (size_t)src * ldx;
    const int part = W / groups;
    for (int g = 0; g < groups; ++g) {
        const int c0 = g * part;
        float ss = 0.f;
        for (int c = threadIdx.x; c < part; c += 256) ss = fmaf(xr[c0 + c], xr[c0 + c], ss);
        ss = warp_sum(ss);
        if (g) __syncthreads();
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) tot += red[w];
        const float inv = 1.f / sqrtf(tot / (float)part + eps);
        for (int c = c0 + threadIdx.x; c < c0 + part; c += 256) {
            const float v = xr[c] * inv;
            store_act(out1, r, c, v * w1[c]);
            if (w2) store_act(out2, r, c, v * w2[c]);
        }
    }
}

__global__ void store_rows_kernel(const float* __restrict__ src, int lds, int W, ActOut dst, int col0) {
    const int r = blockIdx.x;
    for (int c = threadIdx.x; c < W; c += blockDim.x) store_act(dst, r, col0 + c, src[(size_t)r * lds + c]);
}

__global__ void gather_rows_kernel(const float* __restrict__ src, int lds, const int* __restrict__ rows, int W, float* __restrict__ dst, int ldd) {
    const int r = blockIdx.x;
    for (int c = threadIdx.x; c < W; c += blockDim.x) dst[(size_t)r * ldd + c] = src[(size_t)rows[r] * lds + c];
}

// ---------------------------------------------------------------------------------------------------------------- exact linear
// 64 x 64 output tile, 16-wide k-steps, 256 threads x (4 x 4) accumulators; each output element sums its k-steps in order, every
// k-step summed on its own first (a fixed two-level order, the same for every row count).
template <int MODE>
__global__ void __launch_bounds__(256) linear_f32_kernel(const float* __restrict__ A, int lda, const bf16* __restrict__ Wt, int ldw, int M, int N,
                                                         int K, float* __restrict__ C, int ldc, const float* __restrict__ col_scale,
                                                         const float* __restrict__ gate, int ldg, const float* __restrict__ gate_bias) {
    __shared__ float sa[16][64 + 4], sw[16][64 + 4];
    const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64, tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += 16) {
        for (int i = tid; i < 64 * 16; i += 256) {
            const int r = i >> 4, k = i & 15;
            sa[k][r] = (m0 + r < M && k0 + k < K) ? A[(size_t)(m0 + r) * lda + k0 + k] : 0.f;
            sw[k][r] = (n0 + r < N && k0 + k < K) ? __bfloat162float(Wt[(size_t)(n0 + r) * ldw + k0 + k]) : 0.f;
        }
        __syncthreads();
        float part[4][4] = {};                  // the k-step's own sum first, then one addition into the total: rounding grows with 16 + K / 16 terms, not K
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            float av[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { av[i] = sa[k][ty * 4 + i]; wv[i] = sw[k][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) part[i][j] = fmaf(av[i], wv[j], part[i][j]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] += part[i][j];
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
            if (m < M && n < N) {
                float* p = C + (size_t)m * ldc + n;
                float v = acc[i][j];
                if (MODE == LIN_RESID && col_scale) v *= col_scale[n];
                if (MODE == LIN_RESID && gate) v *= 1.f / (1.f + expf(-(gate[(size_t)m * ldg + n] + (gate_bias ? gate_bias[n] : 0.f))));
                *p = (MODE == LIN_RESID) ? *p + v : v;
            }
        }
}

// ---------------------------------------------------------------------------------------------------------------- attention
// One warp per (row, head): q -> rms_norm(q) [* w] * temp(pos), rotated; k -> rms_norm(k) [* w], rotated, into its page; v into its page.
// The rotation turns neighbouring pairs (2i, 2i + 1) of the first rot_dims dimensions by pos * rot_freq[i]; the row's cosines and
// sines are taken once per row, in 64-bit, and shared by its heads.
template <typename KT>
__global__ void attn_prep_kernel(RaggedBatch rb, AttnPrepArgs a) {
    extern __shared__ float rot_cs[];                    // [rot_dims / 2] cos, then sin
    __shared__ float whole[2][8];
    const int r = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int e = rb.row_entry[r], pos = rb.row_pos[r], slot = rb.ent_slot[e];
    const float* row = a.qkv + (size_t)r * a.ld;
    const int nk = a.has_kv ? a.G : 0, nv = (a.has_kv && !a.v_from_k) ? a.G : 0;
    const int nheads = a.H + nk + nv;
    const int nrot = a.rot_dims / 2;
    if (nrot > 0) {
        for (int i = threadIdx.x; i < nrot; i += blockDim.x) {
            double sn, cs;
            sincos((double)pos * a.rot_freq[i], &sn, &cs);
            rot_cs[i] = (float)cs; rot_cs[nrot + i] = (float)sn;
        }
        __syncthreads();
    }
    // one statistic over all query heads and one over all key heads: thread-strided partial sums, warp tree, warps in order
    float inv_whole[2] = {1.f, 1.f};
    if (a.whole_norm && !a.no_norm) {
        for (int which = 0; which < 2; ++which) {
            const int n = which ? nk * a.d : a.H * a.d, off = which ? a.H * a.d : 0;
            float ss = 0.f;
            for (int c = threadIdx.x; c < n; c += blockDim.x) { const float v = row[off + c] + (a.bias ? a.bias[off + c] : 0.f); ss = fmaf(v, v, ss); }
            ss = warp_sum(ss);
            if (lane == 0) whole[which][warp] = ss;
        }
        __syncthreads();
        for (int which = 0; which < 2; ++which) {
            const int n = which ? nk * a.d : a.H * a.d;
            float tot = 0.f;
            for (int w = 0; w < nw; ++w) tot += whole[which][w];
            inv_whole[which] = n > 0 ? 1.f / sqrtf(tot / (float)n + a.eps) : 1.f;
        }
    }
    float temp = 1.f;
    if (a.temp_every > 0) temp = 1.f + a.temp_coef * logf((float)((pos + 1) / a.temp_every) + 1.f);
    const int page = a.has_kv ? a.block_table[(size_t)slot * a.max_pages + pos / KV_PAGE] : 0;
    for (int hh = warp; hh < nheads; hh += nw) {
        if (hh < a.H + nk) {             // q or k head: RMS norm over d (or the row's whole-projection statistic)
            const bool isq = hh < a.H;
            const float* src = row + (size_t)hh * a.d;
            const float* bsrc = a.bias ? a.bias + (size_t)hh * a.d : nullptr;
            const float* nwt = isq ? a.q_norm_w : a.k_norm_w;
            if (nwt && a.whole_norm) nwt += (size_t)(isq ? hh : hh - a.H) * a.d;
            float ss = 0.f;
            for (int c = lane; c < a.d; c += 32) { const float v = src[c] + (bsrc ? bsrc[c] : 0.f); ss += v * v; }
            ss = warp_sum(ss);
            float inv = a.no_norm ? 1.f : (a.whole_norm ? inv_whole[isq ? 0 : 1] : 1.f / sqrtf(ss / (float)a.d + a.eps)) * (isq ? temp : 1.f);
            if (isq && a.q_head_scale) inv *= a.q_head_scale[hh];
            KT* dst = nullptr; KT* dstv = nullptr;
            if (!isq) {
                const size_t at = ((size_t)page * a.G + (hh - a.H)) * KV_PAGE + (pos % KV_PAGE);
                dst = (KT*)a.k_pool + at * a.d;
                if (a.v_from_k) dstv = (KT*)a.v_pool + at * a.dv;
            }
            // a lane owns the pairs (2i, 2i + 1), i = lane, lane + 32, ...: both halves of a rotated pair are in one thread
            for (int c = 2 * lane; c < a.d; c += 64) {
                const float u0 = src[c] + (bsrc ? bsrc[c] : 0.f), v0 = (c + 1 < a.d) ? src[c + 1] + (bsrc ? bsrc[c + 1] : 0.f) : 0.f;
                if (dstv) {               // the value is the key as projected
                    kv_store<KT>(dstv + c, u0, a.kv_lo_off);
                    if (c + 1 < a.d) kv_store<KT>(dstv + c + 1, v0, a.kv_lo_off);
                }
                float u = u0 * inv, v = v0 * inv;
                if (nwt) { u *= nwt[c]; if (c + 1 < a.d) v *= nwt[c + 1]; }
                if (c + 1 < a.rot_dims) {
                    const float cs = rot_cs[c >> 1], sn = rot_cs[nrot + (c >> 1)];
                    const float u2 = u * cs - v * sn, v2 = v * cs + u * sn;
                    u = u2; v = v2;
                }
                if (isq) {
                    store_act(a.q_out, r, hh * a.d + c, u);
                    if (c + 1 < a.d) store_act(a.q_out, r, hh * a.d + c + 1, v);
                } else {
                    kv_store<KT>(dst + c, u, a.kv_lo_off);
                    if (c + 1 < a.d) kv_store<KT>(dst + c + 1, v, a.kv_lo_off);
                }
            }
        } else {
            const int g = hh - a.H - a.G;
            const size_t off = (size_t)(a.H + a.G) * a.d + (size_t)g * a.dv;
            const float* src = row + off;
            const float* bsrc = a.bias ? a.bias + off : nullptr;
            KT* dst = (KT*)a.v_pool + (((size_t)page * a.G + g) * KV_PAGE + (pos % KV_PAGE)) * a.dv;
            float inv = 1.f;
            if (a.v_unit) {
                float ss = 0.f;
                for (int c = lane; c < a.dv; c += 32) { const float v = src[c] + (bsrc ? bsrc[c] : 0.f); ss += v * v; }
                inv = 1.f / sqrtf(warp_sum(ss) / (float)a.dv + a.eps);
            }
            for (int c = lane; c < a.dv; c += 32) kv_store<KT>(dst + c, (src[c] + (bsrc ? bsrc[c] : 0.f)) * inv, a.kv_lo_off);
        }
    }
}

constexpr int ATT_WARPS = 4;
constexpr int ATT_MAXC = 8;      // value columns per lane: dv <= 256

// Block = (row, group of up to REP query heads that share one key/value head, split).  Its warps walk 32-key tiles of the split's
// key range: one key per lane for the scores -- the key is fetched and widened once and multiplied into every query head of the
// group -- then eight contiguous value columns per lane for the weighted sums, online softmax per warp and head; warps, then
// splits, merge in a fixed order.  Widths that are not multiples of 8 take the element-wise loads.
template <typename KT> __device__ __forceinline__ void kv_load8(const KT* p, long long lo, float* v);
template <> __device__ __forceinline__ void kv_load8<float>(const float* p, long long, float* v) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <> __device__ __forceinline__ void kv_load8<bf16>(const bf16* p, long long lo, float* v) {
    const uint4 h = *reinterpret_cast<const uint4*>(p);
    v[0] = bf16lo(h.x); v[1] = bf16hi(h.x); v[2] = bf16lo(h.y); v[3] = bf16hi(h.y);
    v[4] = bf16lo(h.z); v[5] = bf16hi(h.z); v[6] = bf16lo(h.w); v[7] = bf16hi(h.w);
    if (lo) {
        const uint4 l = *reinterpret_cast<const uint4*>(p + lo);
        v[0] += bf16lo(l.x); v[1] += bf16hi(l.x); v[2] += bf16lo(l.y); v[3] += bf16hi(l.y);
        v[4] += bf16lo(l.z); v[5] += bf16hi(l.z); v[6] += bf16lo(l.w); v[7] += bf16hi(l.w);
    }
}
template <typename KT, int REP, bool STAGE>
__global__ void __launch_bounds__(ATT_WARPS * 32) sink_attention_kernel(RaggedBatch rb, SinkAttnArgs a) {
    constexpr bool stage = STAGE;
    extern __shared__ __align__(16) float smem[];
    const int d = a.d, dv = a.dv, rep = a.H / a.G, nb = (rep + REP - 1) / REP;
    float* sq = smem;                                   // [REP][d]
    float* wm = sq + REP * d;                           // [ATT_WARPS][REP] m, then l, then [ATT_WARPS][REP][dv] acc
    float* wl = wm + ATT_WARPS * REP;
    float* wa = wl + ATT_WARPS * REP;
    const int r = blockIdx.x, sp = blockIdx.z, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = blockIdx.y / nb, h0 = g * rep + (blockIdx.y % nb) * REP, nh = min(REP, (g + 1) * rep - h0);
    const int e = rb.row_entry[r], pos = rb.row_pos[r], slot = rb.ent_slot[e];
    const int* bt = a.block_table + (size_t)slot * a.max_pages;
    for (int i = threadIdx.x; i < nh * d; i += blockDim.x) sq[i] = a.q[(size_t)r * a.ldq + (size_t)h0 * d + i] * a.scale;
    __syncthreads();
    const int nkeys = pos + 1;
    const int key0 = (a.window > 0 && nkeys > a.window) ? nkeys - a.window : 0;      // first key the row sees
    const int t0 = key0 / 32;                            // (its tile holds at least that key: no tile is hidden entirely)
    const int ntiles = (nkeys + 31) / 32, per = (ntiles - t0 + a.nsplit - 1) / a.nsplit;
    const int t_lo = t0 + sp * per, t_hi = min(ntiles, t_lo + per);
    float m[REP], l[REP], acc[REP][ATT_MAXC];
#pragma unroll
    for (int q = 0; q < REP; ++q) {
        m[q] = -INFINITY; l[q] = 0.f;
#pragma unroll
        for (int c = 0; c < ATT_MAXC; ++c) acc[q][c] = 0.f;
    }
    const bool kvec = (d & 7) == 0, vvec = (dv & 7) == 0;
    // STAGE (widths that allow 16-byte copies, room in shared memory, a small launch): a warp first brings its whole tile -- 32 key rows and
    // 32 value rows, every plane -- into its own shared-memory patch with one burst of cp.async, so the tile costs one trip to memory
    // instead of a dozen dependent load rounds; rows are padded by 16 bytes, which spreads a lane-per-row access over all banks.
    // The arithmetic and its order are the same either way.
    // kv_shared (one pool serves as keys and as values, d == dv): the staged key rows are the value rows too -- one copy, half the patch.
    const bool one_copy = stage && a.kv_shared;
    const int ks_e = stage ? d + 16 / (int)sizeof(KT) : d, vs_e = stage ? dv + 16 / (int)sizeof(KT) : dv;      // row strides (elements)
    const int planes = (sizeof(KT) == 2 && a.kv_lo_off) ? 2 : 1;
    KT* kst = nullptr; KT* vst = nullptr;
    if (stage) {
        KT* all = reinterpret_cast<KT*>(wa + (size_t)ATT_WARPS * REP * dv + ((4 - ((REP * d + 2 * ATT_WARPS * REP + ATT_WARPS * REP * dv) & 3)) & 3));
        kst = all + (size_t)warp * 32 * planes * (one_copy ? ks_e : ks_e + vs_e);
        vst = one_copy ? kst : kst + (size_t)32 * planes * ks_e;
    }
    const long long klo = !stage ? a.kv_lo_off : planes == 2 ? (long long)32 * ks_e : 0, vlo = !stage ? a.kv_lo_off : planes == 2 ? (long long)32 * vs_e : 0;
    for (int t = t_lo + warp; t < t_hi; t += ATT_WARPS) {
        const int j = t * 32 + lane;
        const int pg = bt[(t * 32) / KV_PAGE];           // a 32-key tile never straddles a 64-token page
        const size_t base = ((size_t)pg * a.G + g) * KV_PAGE + ((t * 32) % KV_PAGE);
        const int cnt = min(32, nkeys - t * 32);
        if (stage) {
            __syncwarp();                                 // the patch's last readers are done
            const int kc = d * (int)sizeof(KT) / 16, vc = dv * (int)sizeof(KT) / 16;      // 16-byte pieces per row
            for (int pl = 0; pl < planes; ++pl) {
                const KT* ksrc = (const KT*)a.k_pool + base * d + (pl ? a.kv_lo_off : 0);
                const KT* vsrc = (const KT*)a.v_pool + base * dv + (pl ? a.kv_lo_off : 0);
                for (int i = lane; i < cnt * kc; i += 32) {
                    const int row = i / kc, ch = i % kc;
                    cp_async16s(reinterpret_cast<unsigned char*>(kst + (size_t)pl * 32 * ks_e + (size_t)row * ks_e) + ch * 16,
                                reinterpret_cast<const unsigned char*>(ksrc + (size_t)row * d) + ch * 16);
                }
                for (int i = lane; i < (one_copy ? 0 : cnt * vc); i += 32) {
                    const int row = i / vc, ch = i % vc;
                    cp_async16s(reinterpret_cast<unsigned char*>(vst + (size_t)pl * 32 * vs_e + (size_t)row * vs_e) + ch * 16,
                                reinterpret_cast<const unsigned char*>(vsrc + (size_t)row * dv) + ch * 16);
                }
            }
            asm volatile("cp.async.commit_group;\n cp.async.wait_group 0;" ::: "memory");
            __syncwarp();
        }
        float sc[REP];
#pragma unroll
        for (int q = 0; q < REP; ++q) sc[q] = 0.f;
        const bool seen = j < nkeys && j >= key0;
        if (seen) {
            const KT* kr = stage ? kst + (size_t)lane * ks_e : (const KT*)a.k_pool + (base + lane) * d;
            if (kvec) {
                // UN pieces of the key row are requested before the first is used: the loop is bound by memory latency, not by arithmetic
                constexpr int UN = REP <= 2 ? 4 : 2;
                for (int c0 = 0; c0 < d; c0 += 8 * UN) {
                    float kf[UN][8];
#pragma unroll
                    for (int u = 0; u < UN; ++u) if (c0 + 8 * u < d) kv_load8<KT>(kr + c0 + 8 * u, klo, kf[u]);
#pragma unroll
                    for (int u = 0; u < UN; ++u) {
                        const int c = c0 + 8 * u;
                        if (c >= d) break;
#pragma unroll
                        for (int q = 0; q < REP; ++q) {
                            if (q < nh) {
                                const float4 qa = *reinterpret_cast<const float4*>(sq + q * d + c), qb = *reinterpret_cast<const float4*>(sq + q * d + c + 4);
                                float x = sc[q];
                                x = fmaf(qa.x, kf[u][0], x); x = fmaf(qa.y, kf[u][1], x); x = fmaf(qa.z, kf[u][2], x); x = fmaf(qa.w, kf[u][3], x);
                                x = fmaf(qb.x, kf[u][4], x); x = fmaf(qb.y, kf[u][5], x); x = fmaf(qb.z, kf[u][6], x); x = fmaf(qb.w, kf[u][7], x);
                                sc[q] = x;
                            }
                        }
                    }
                }
            } else {
                for (int c = 0; c < d; ++c) {
                    const float kf = kv_load<KT>(kr + c, a.kv_lo_off);
#pragma unroll
                    for (int q = 0; q < REP; ++q) if (q < nh) sc[q] = fmaf(sq[q * d + c], kf, sc[q]);
                }
            }
        }
        if (seen && (a.softcap > 0.f || a.dist_r1 || a.dist_table)) {       // cap, then the distance terms (f32, the row's own distance to the key)
            const int dist = pos - j;
#pragma unroll
            for (int q = 0; q < REP; ++q) {
                if (q < nh) {
                    float x = sc[q];
                    if (a.softcap > 0.f) x = a.softcap * tanhf(x / a.softcap);
                    if (a.dist_r1) x -= a.dist_r1[h0 + q] * log1pf(a.dist_r2[h0 + q] * (float)dist);
                    if (a.dist_table) x += a.dist_table[(size_t)(h0 + q) * a.dist_rows + min(dist, a.dist_rows - 1)];
                    sc[q] = x;
                }
            }
        }
        float p[REP];
#pragma unroll
        for (int q = 0; q < REP; ++q) {
            const float sv = seen ? sc[q] : -INFINITY;
            const float mn = fmaxf(m[q], warp_max(sv));
            const float corr = (m[q] == -INFINITY) ? 0.f : __expf(m[q] - mn);
            p[q] = seen ? __expf(sv - mn) : 0.f;
            l[q] = l[q] * corr + warp_sum(p[q]);
#pragma unroll
            for (int c = 0; c < ATT_MAXC; ++c) acc[q][c] *= corr;
            m[q] = mn;
        }
        const KT* vb = stage ? vst : (const KT*)a.v_pool + base * dv;
        if (vvec) {
            const bool mine = 8 * lane < dv;
            constexpr int VN = REP <= 2 ? 4 : 2;              // value rows in flight
            for (int j0 = 0; j0 < cnt; j0 += VN) {
                float v[VN][8];
#pragma unroll
                for (int u = 0; u < VN; ++u) if (mine && j0 + u < cnt) kv_load8<KT>(vb + (size_t)(j0 + u) * vs_e + 8 * lane, vlo, v[u]);
#pragma unroll
                for (int u = 0; u < VN; ++u) {
                    const int jj = j0 + u;                    // (uniform over the warp)
                    if (jj >= cnt) break;
#pragma unroll
                    for (int q = 0; q < REP; ++q) {
                        const float pj = __shfl_sync(0xffffffffu, p[q], jj);
                        if (mine && q < nh) {
#pragma unroll
                            for (int c = 0; c < 8; ++c) acc[q][c] = fmaf(pj, v[u][c], acc[q][c]);
                        }
                    }
                }
            }
        } else {
            for (int jj = 0; jj < cnt; ++jj) {
                float v[ATT_MAXC];
#pragma unroll
                for (int c = 0; c < ATT_MAXC; ++c) { const int col = lane + 32 * c; v[c] = col < dv ? kv_load<KT>(vb + (size_t)jj * dv + col, a.kv_lo_off) : 0.f; }
#pragma unroll
                for (int q = 0; q < REP; ++q) {
                    const float pj = __shfl_sync(0xffffffffu, p[q], jj);
#pragma unroll
                    for (int c = 0; c < ATT_MAXC; ++c) acc[q][c] = fmaf(pj, v[c], acc[q][c]);
                }
            }
        }
    }
    // merge the warps in warp order, head by head
#pragma unroll
    for (int q = 0; q < REP; ++q) {
        if (q < nh) {
            if (lane == 0) { wm[warp * REP + q] = m[q]; wl[warp * REP + q] = l[q]; }
#pragma unroll
            for (int c = 0; c < ATT_MAXC; ++c) { const int col = vvec ? 8 * lane + c : lane + 32 * c; if (col < dv) wa[((size_t)warp * REP + q) * dv + col] = acc[q][c]; }
        }
    }
    __syncthreads();
    const bool last = a.nsplit == 1;
    for (int q = 0; q < nh; ++q) {
        const int h = h0 + q;
        float M = -INFINITY;
        for (int w = 0; w < ATT_WARPS; ++w) M = fmaxf(M, wm[w * REP + q]);
        const float sink = (last && a.sink) ? a.sink[h] : -INFINITY;
        const float Mx = fmaxf(M, sink);
        float Lsum = (sink == -INFINITY) ? 0.f : __expf(sink - Mx);
        float wsc[ATT_WARPS];
        for (int w = 0; w < ATT_WARPS; ++w) { wsc[w] = (wm[w * REP + q] == -INFINITY) ? 0.f : __expf(wm[w * REP + q] - Mx); Lsum += wl[w * REP + q] * wsc[w]; }
        for (int col = threadIdx.x; col < dv; col += blockDim.x) {
            float o = 0.f;
            for (int w = 0; w < ATT_WARPS; ++w) o += wa[((size_t)w * REP + q) * dv + col] * wsc[w];
            if (last) store_act(a.out, r, h * dv + col, o / Lsum * (a.gate ? 1.f / (1.f + __expf(-a.gate[(size_t)r * a.ldg + h * dv + col])) : 1.f));
            else a.part[(((size_t)r * a.H + h) * a.nsplit + sp) * (dv + 2) + 2 + col] = o;
        }
        if (!last && threadIdx.x == 0) {
            float* pp = a.part + (((size_t)r * a.H + h) * a.nsplit + sp) * (dv + 2);
            pp[0] = Mx; pp[1] = Lsum;          // (no sink yet: Mx == M, possibly -inf for an empty split)
        }
    }
}

__global__ void sink_attention_merge_kernel(SinkAttnArgs a) {
    __shared__ float wgt[64];
    __shared__ float Ls;
    const int r = blockIdx.x, h = blockIdx.y, dv = a.dv, ns = a.nsplit;           // nsplit <= 64
    const float* pp = a.part + ((size_t)r * a.H + h) * ns * (dv + 2);
    const float sink = a.sink ? a.sink[h] : -INFINITY;
    if (threadIdx.x < 32) {                 // one warp: the maximum over the splits and the sink, then each split's weight, in split order
        const int lane = threadIdx.x;
        const float m0 = lane < ns ? pp[(size_t)lane * (dv + 2)] : -INFINITY, m1 = lane + 32 < ns ? pp[(size_t)(lane + 32) * (dv + 2)] : -INFINITY;
        const float Mx = fmaxf(warp_max(fmaxf(m0, m1)), sink);
        const float w0 = m0 == -INFINITY ? 0.f : __expf(m0 - Mx), w1 = m1 == -INFINITY ? 0.f : __expf(m1 - Mx);
        wgt[lane] = w0; wgt[lane + 32] = w1;
        const float l0 = lane < ns ? pp[(size_t)lane * (dv + 2) + 1] * w0 : 0.f, l1 = lane + 32 < ns ? pp[(size_t)(lane + 32) * (dv + 2) + 1] * w1 : 0.f;
        const float L = warp_sum(l0 + l1) + (sink == -INFINITY ? 0.f : __expf(sink - Mx));
        if (lane == 0) Ls = L;
    }
    __syncthreads();
    const float invL = 1.f / Ls;
    for (int col = threadIdx.x; col < dv; col += blockDim.x) {
        float o = 0.f;
#pragma unroll 4
        for (int sp = 0; sp < ns; ++sp) o = fmaf(pp[(size_t)sp * (dv + 2) + 2 + col], wgt[sp], o);
        store_act(a.out, r, h * dv + col, o * invL * (a.gate ? 1.f / (1.f + __expf(-a.gate[(size_t)r * a.ldg + h * dv + col])) : 1.f));
    }
}

// ---------------------------------------------------------------------------------------------------------------- Mamba-2
// Causal depthwise convolution over the x | B | C columns + SiLU.  The taps that reach before the entry's first row read the
// sequence's carried window (zeros for a new sequence).
__global__ void conv_silu_kernel(RaggedBatch rb, Mamba2Args a, int C, int col0) {
    const int r = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int e = rb.row_entry[r], i = r - rb.ent_row0[e], slot = rb.ent_slot[e], taps = a.taps;
    const float* win = a.conv_state + (size_t)slot * (taps - 1) * C;
    float acc = a.conv_b[c];
    for (int k = 0; k < taps; ++k) {
        const int back = taps - 1 - k;                   // this tap reads the input `back` tokens ago
        const float u = (i - back >= 0) ? a.proj[(size_t)(r - back) * a.ldp + col0 + c] : win[(size_t)(taps - 1 + i - back) * C + c];
        acc = fmaf(a.conv_w[(size_t)c * taps + k], u, acc);
    }
    a.xbc[(size_t)r * C + c] = acc / (1.f + __expf(-acc));
}
// Every entry one token (decode): the convolution and the window shift in one pass; thread = (entry, channel) owns its window column.
__global__ void conv_step_kernel(RaggedBatch rb, Mamba2Args a, int C, int col0) {
    const int e = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int r = rb.ent_row0[e], slot = rb.ent_slot[e], taps = a.taps;
    float* win = a.conv_state + (size_t)slot * (taps - 1) * C;
    const float u = a.proj[(size_t)r * a.ldp + col0 + c];
    float acc = fmaf(a.conv_w[(size_t)c * taps + taps - 1], u, a.conv_b[c]);
    for (int k = 0; k < taps - 1; ++k) {
        const float w = win[(size_t)k * C + c];
        acc = fmaf(a.conv_w[(size_t)c * taps + k], w, acc);
        if (k > 0) win[(size_t)(k - 1) * C + c] = w;
    }
    if (taps > 1) win[(size_t)(taps - 2) * C + c] = u;
    a.xbc[(size_t)r * C + c] = acc / (1.f + __expf(-acc));
}
// New window = the last taps-1 inputs of the sequence (older ones shift down when the entry is shorter than the window).
__global__ void conv_window_kernel(RaggedBatch rb, Mamba2Args a, int C, int col0) {
    const int e = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int len = rb.ent_len[e], r0 = rb.ent_row0[e], slot = rb.ent_slot[e], nwin = a.taps - 1;
    float* win = a.conv_state + (size_t)slot * nwin * C;
    for (int i = 0; i < nwin; ++i) {
        const int src = len - nwin + i;                  // index among this entry's rows
        win[(size_t)i * C + c] = (src >= 0) ? a.proj[(size_t)(r0 + src) * a.ldp + col0 + c] : win[(size_t)(i + len) * C + c];
    }
}

// Selective scan.  Block = (entry, head, slice of SSD_COLS value columns); thread (p, ns) owns state rows n = ns, ns + 8, ... of
// column p in registers for the whole portion.  The recurrence itself is one FMA deep per token; what would serialise it is the
// operand fetch, so the step inputs (x slice, B, C, dt) of SSD_CH tokens at a time are staged in shared memory with cp.async,
// double-buffered: chunk c + 1 is in flight while chunk c is consumed.  dt = softplus(.) and the decay exp(-exp(A) dt) are
// computed once per token, in f32, when its chunk lands.
constexpr int SSD_NS = 8, SSD_MAXR = 32, SSD_COLS = 16, SSD_CH = 16;      // N <= 256; 16 columns x 8 = 128 threads per block: one warp per scheduler, many blocks
// Staged layout of one token: x slice [SSD_COLS] | B | C | dt, pad.  Thread ns owns the CONTIGUOUS state rows ns * R .. ns * R + R - 1,
// so it reads its B and C values as float4; every R-run is followed by 4 pad floats, which spreads the eight runs of a warp over
// all banks.
__host__ __device__ inline int ssd_idx(int n, int R) { return n + 4 * (n / R); }
__host__ __device__ inline int ssd_npad(int N, int R) { (void)N; return 8 * (R + 4); }      // all eight runs, whatever N: no bounds checks in the loop
// Long portions are cut into SSD_SEGS segments that run side by side (the scan has one resident warp per scheduler and waits on
// its own dependent chain most of the time): the recurrence is linear with a SCALAR decay per head and token, so
//   S_end(segment) = (product of the segment's decays) * S_start + S_local(segment run from zero).
// MODE 1 runs every segment from zero and leaves S_local and the decay product; ssd_seg_prefix_kernel turns them into each segment's
// start state (and the sequence's new state); MODE 2 is the scan proper from those start states.  MODE 0 = one segment, everything.
constexpr int SSD_SEGS = 4, SSD_SEG_MIN = 512;              // segmented from this many rows in the longest entry
__host__ __device__ inline int ssd_seg_len(int len) { return ((len + SSD_SEGS - 1) / SSD_SEGS + SSD_CH - 1) / SSD_CH * SSD_CH; }
template <int SSD_R, int MODE>                               // state rows per thread: ceil(N / 8) rounded up to 4, 8, 16 or 32
__global__ void __launch_bounds__(SSD_COLS * SSD_NS) ssd_scan_kernel(RaggedBatch rb, Mamba2Args a, int C) {
    extern __shared__ __align__(16) float ssm_s[];
    const int e = MODE == 0 ? blockIdx.x : blockIdx.x / SSD_SEGS, seg = MODE == 0 ? 0 : blockIdx.x % SSD_SEGS;
    const int h = blockIdx.y, ns = threadIdx.x & (SSD_NS - 1), pl = threadIdx.x / SSD_NS;
    const int p0 = blockIdx.z * SSD_COLS, p = p0 + pl;
    const int P = a.P, N = a.N, inner = a.heads * P, g = h / (a.heads / a.groups);
    const bool live = p < P;
    const int full_len = rb.ent_len[e], slot = rb.ent_slot[e];
    const int seg_len = MODE == 0 ? full_len : ssd_seg_len(full_len), seg0 = seg * seg_len;
    if (seg0 >= full_len) return;                             // (a short entry has fewer segments)
    const int len = min(seg_len, full_len - seg0), r0 = rb.ent_row0[e] + seg0;
    const int ncol = min(SSD_COLS, P - p0);
    const int NP = ssd_npad(N, SSD_R), per_tok = SSD_COLS + 2 * NP + 4;
    float* stage[2] = {ssm_s, ssm_s + SSD_CH * per_tok};
    float* sdt = ssm_s + 2 * SSD_CH * per_tok;                // [SSD_CH] dt, [SSD_CH] decay
    float* S = MODE == 0 ? a.ssm_state + (((size_t)slot * a.heads + h) * N) * P
                         : a.seg_state + ((((size_t)e * SSD_SEGS + seg) * a.heads + h) * N) * P;
    const int n0 = ns * SSD_R;
    // rows past N and tokens past the portion's end multiply zeros: the stages start zeroed and only real values are ever copied in
    for (int i = threadIdx.x; i < 2 * SSD_CH * per_tok; i += blockDim.x) ssm_s[i] = 0.f;
    __syncthreads();
    float s[SSD_R];
#pragma unroll
    for (int i = 0; i < SSD_R; ++i) s[i] = (MODE != 1 && n0 + i < N && live) ? S[(size_t)(n0 + i) * P + p] : 0.f;
    float dprod = 1.f;                                        // MODE 1, thread 0: product of the segment's decays
    const float negA = -__expf(a.A_log[h]), Dh = a.D[h], dtb = a.dt_bias[h];
    const int dtcol = 2 * inner + 2 * a.groups * N + h;
    const int src_tok = SSD_COLS + 2 * N + 1;
    // 16-byte copies when every segment starts on a 16-byte boundary (the usual geometry), 4-byte copies otherwise
    const bool wide = ((N | P | inner | C | a.ldp | (a.groups * N)) & 3) == 0;
    auto fetch = [&](int c, float* dst) {                     // tokens [c * SSD_CH, ...) of the portion
        const int t0 = c * SSD_CH, nt = min(SSD_CH, len - t0);
        if (wide) {                                           // 8 threads per token: x (4 pieces), B and C (N / 4 pieces each), dt
            const int t = threadIdx.x >> 3, q = threadIdx.x & 7, nq = N >> 2;
            if (t < nt) {
                const float* row = a.xbc + (size_t)(r0 + t0 + t) * C;
                float* d0 = dst + t * per_tok;
                for (int k = q; k < SSD_COLS / 4 + 2 * nq; k += 8) {
                    if (k < SSD_COLS / 4) { if (4 * k < ncol) cp_async16s(d0 + 4 * k, row + h * P + p0 + 4 * k); }
                    else if (k < SSD_COLS / 4 + nq) { const int n = 4 * (k - SSD_COLS / 4); cp_async16s(d0 + SSD_COLS + ssd_idx(n, SSD_R), row + inner + g * N + n); }
                    else { const int n = 4 * (k - SSD_COLS / 4 - nq); cp_async16s(d0 + SSD_COLS + NP + ssd_idx(n, SSD_R), row + inner + (a.groups + g) * N + n); }
                }
                if (q == 0) cp_async4(d0 + SSD_COLS + 2 * NP, a.proj + (size_t)(r0 + t0 + t) * a.ldp + dtcol);
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            return;
        }
        for (int i = threadIdx.x; i < nt * src_tok; i += blockDim.x) {
            const int t = i / src_tok, j = i - t * src_tok, r = r0 + t0 + t;
            const float* src;
            int d;
            if (j < SSD_COLS) { if (j >= ncol) continue; src = a.xbc + (size_t)r * C + h * P + p0 + j; d = j; }
            else if (j < SSD_COLS + N) { const int n = j - SSD_COLS; src = a.xbc + (size_t)r * C + inner + g * N + n; d = SSD_COLS + ssd_idx(n, SSD_R); }
            else if (j < SSD_COLS + 2 * N) { const int n = j - SSD_COLS - N; src = a.xbc + (size_t)r * C + inner + (a.groups + g) * N + n; d = SSD_COLS + NP + ssd_idx(n, SSD_R); }
            else { src = a.proj + (size_t)r * a.ldp + dtcol; d = SSD_COLS + 2 * NP; }
            cp_async4(dst + t * per_tok + d, src);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const int nch = (len + SSD_CH - 1) / SSD_CH;
    fetch(0, stage[0]);
    for (int c = 0; c < nch; ++c) {
        if (c + 1 < nch) { fetch(c + 1, stage[(c + 1) & 1]); asm volatile("cp.async.wait_group 1;" ::: "memory"); }
        else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        const float* st = stage[c & 1];
        const int nt = min(SSD_CH, len - c * SSD_CH);
        if (threadIdx.x < SSD_CH) {
            const float z = st[threadIdx.x * per_tok + SSD_COLS + 2 * NP] + dtb;
            const float dt = threadIdx.x < nt ? ((z > 20.f) ? z : log1pf(__expf(z))) : 0.f;      // past the end: the state stands still
            sdt[threadIdx.x] = dt; sdt[SSD_CH + threadIdx.x] = __expf(negA * dt);
        }
        __syncthreads();
        if (MODE == 1 && threadIdx.x == 0) for (int t = 0; t < nt; ++t) dprod *= sdt[SSD_CH + t];
        const int tmax = (nt + 3) & ~3;                       // whole groups of four: the padding tokens leave the state as it is
#pragma unroll 4
        for (int t = 0; t < tmax; ++t) {
            const float* tk = st + t * per_tok;
            const float dt = sdt[t], decay = sdt[SSD_CH + t];
            const float xv = live ? tk[pl] : 0.f;
            const float4* B4 = reinterpret_cast<const float4*>(tk + SSD_COLS + ssd_idx(n0, SSD_R));
            const float4* C4 = reinterpret_cast<const float4*>(tk + SSD_COLS + NP + ssd_idx(n0, SSD_R));
            const float dx = dt * xv;
            if (MODE == 1) {                                  // state only
#pragma unroll
                for (int i = 0; i < SSD_R / 4; ++i) {
                    const float4 b = B4[i];
                    s[4 * i] = fmaf(decay, s[4 * i], b.x * dx); s[4 * i + 1] = fmaf(decay, s[4 * i + 1], b.y * dx);
                    s[4 * i + 2] = fmaf(decay, s[4 * i + 2], b.z * dx); s[4 * i + 3] = fmaf(decay, s[4 * i + 3], b.w * dx);
                }
                continue;
            }
            float y0 = 0.f, y1 = 0.f;
#pragma unroll
            for (int i = 0; i < SSD_R / 4; ++i) {
                const float4 b = B4[i], cc = C4[i];
                { s[4 * i]     = fmaf(decay, s[4 * i],     b.x * dx); y0 = fmaf(s[4 * i],     cc.x, y0); }
                { s[4 * i + 1] = fmaf(decay, s[4 * i + 1], b.y * dx); y1 = fmaf(s[4 * i + 1], cc.y, y1); }
                { s[4 * i + 2] = fmaf(decay, s[4 * i + 2], b.z * dx); y0 = fmaf(s[4 * i + 2], cc.z, y0); }
                { s[4 * i + 3] = fmaf(decay, s[4 * i + 3], b.w * dx); y1 = fmaf(s[4 * i + 3], cc.w, y1); }
            }
            float y = y0 + y1;
#pragma unroll
            for (int o = SSD_NS / 2; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
            if (ns == 0 && live && t < nt) a.y[(size_t)(r0 + c * SSD_CH + t) * inner + h * P + p] = y + Dh * xv;
        }
        __syncthreads();                                      // the stage is free for chunk c + 2
    }
    if (MODE == 2) return;                                    // the prefix kernel already wrote the sequence's new state
#pragma unroll
    for (int i = 0; i < SSD_R; ++i) if (n0 + i < N && live) S[(size_t)(n0 + i) * P + p] = s[i];
    if (MODE == 1 && threadIdx.x == 0 && blockIdx.z == 0) a.seg_decay[((size_t)e * SSD_SEGS + seg) * a.heads + h] = dprod;
}
// Start state of every segment, in order: seg_state[k] holds S_local on entry and S_start(k) on exit; the slot gets the end state.
__global__ void ssd_seg_prefix_kernel(RaggedBatch rb, Mamba2Args a) {
    const int e = blockIdx.x, h = blockIdx.y, np = a.N * a.P;
    const int len = rb.ent_len[e], slot = rb.ent_slot[e], nseg = (len + ssd_seg_len(len) - 1) / ssd_seg_len(len);
    float* S = a.ssm_state + ((size_t)slot * a.heads + h) * np;
    for (int i = blockIdx.z * blockDim.x + threadIdx.x; i < np; i += gridDim.z * blockDim.x) {
        float cur = S[i];
        for (int k = 0; k < nseg; ++k) {
            float* loc = a.seg_state + (((size_t)e * SSD_SEGS + k) * a.heads + h) * np + i;
            const float l = *loc;
            *loc = cur;
            cur = fmaf(a.seg_decay[((size_t)e * SSD_SEGS + k) * a.heads + h], cur, l);
        }
        S[i] = cur;
    }
}

// out = unit_rms_per_group(y * silu(z)) * w : block per (row, group)
__global__ void gated_group_rms_kernel(Mamba2Args a) {
    __shared__ float scratch[32];
    const int r = blockIdx.x, gi = blockIdx.y, inner = a.heads * a.P, gs = inner / a.norm_groups;
    const float* y = a.y + (size_t)r * inner + gi * gs;
    const float* z = a.proj + (size_t)r * a.ldp + gi * gs;
    float ss = 0.f;
    for (int c = threadIdx.x; c < gs; c += blockDim.x) { const float zz = z[c], v = y[c] * (zz / (1.f + __expf(-zz))); ss += v * v; }
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)gs + a.eps);
    for (int c = threadIdx.x; c < gs; c += blockDim.x) {
        const float zz = z[c], v = y[c] * (zz / (1.f + __expf(-zz)));
        store_act(a.out, r, gi * gs + c, v * inv * a.norm_w[gi * gs + c]);
    }
}

// ---------------------------------------------------------------------------------------------------------------- feed-forwards
__global__ void clamped_glu_kernel(const float* __restrict__ gu, int ld, int stride, int up_off, int F, float limit, ActOut out) {
    const int r = blockIdx.y, j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= F) return;
    const float g = fminf(gu[(size_t)r * ld + (size_t)j * stride], limit);
    const float u = fminf(fmaxf(gu[(size_t)r * ld + (size_t)j * stride + up_off], -limit), limit);
    store_act(out, r, j, g / (1.f + __expf(-1.702f * g)) * (u + 1.f));
}

__global__ void silu_glu_kernel(const float* __restrict__ gu, int ld, int F, ActOut out, float limit) {
    const int r = blockIdx.y, j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= F) return;
    store_act(out, r, j, glu_pair_f(gu[(size_t)r * ld + 2 * j], gu[(size_t)r * ld + 2 * j + 1], limit < 0.f ? limit : 0.f));
}

// Router logits of one row by one warp: NB experts at a time share the loads of the f32 row; a lane owns 8 neighbouring columns per
// 256-column step (one 16-byte load of each bf16 weight row, two of the f32 row), sums them in column order into one accumulator
// per expert, and the lanes meet in warp_sum's tree -- the same order for every row, few or many in the step.  `vec` = the width
// and the leading dimensions allow the 16-byte loads; otherwise lanes stride single columns.
template <int NB>
__device__ __forceinline__ void router_dots(const float* __restrict__ h, const bf16* __restrict__ w, int ldw, int W, int ne, int lane, bool vec, float* out) {
    float acc[NB];
#pragma unroll
    for (int i = 0; i < NB; ++i) acc[i] = 0.f;
    if (vec) {
        for (int k = lane * 8; k < W; k += 256) {
            const float4 x0 = *reinterpret_cast<const float4*>(h + k), x1 = *reinterpret_cast<const float4*>(h + k + 4);
#pragma unroll
            for (int i = 0; i < NB; ++i) {
                if (i < ne) {
                    const uint4 ww = *reinterpret_cast<const uint4*>(w + (size_t)i * ldw + k);
                    float a = acc[i];
                    a = fmaf(bf16lo(ww.x), x0.x, a); a = fmaf(bf16hi(ww.x), x0.y, a); a = fmaf(bf16lo(ww.y), x0.z, a); a = fmaf(bf16hi(ww.y), x0.w, a);
                    a = fmaf(bf16lo(ww.z), x1.x, a); a = fmaf(bf16hi(ww.z), x1.y, a); a = fmaf(bf16lo(ww.w), x1.z, a); a = fmaf(bf16hi(ww.w), x1.w, a);
                    acc[i] = a;
                }
            }
        }
    } else {
        for (int k = lane; k < W; k += 32) {
            const float x = h[k];
#pragma unroll
            for (int i = 0; i < NB; ++i) if (i < ne) acc[i] = fmaf(x, __bfloat162float(w[(size_t)i * ldw + k]), acc[i]);
        }
    }
#pragma unroll
    for (int i = 0; i < NB; ++i) out[i] = warp_sum(acc[i]);
}
__device__ __forceinline__ bool router_vec_ok(int W, int ldw, int ldh) { return (W & 7) == 0 && (ldw & 7) == 0 && (ldh & 3) == 0; }

// Many rows: one warp per row, four experts per pass over the row (which stays in L1).
__global__ void __launch_bounds__(256) router_logits_kernel(MoeArgs a, const bf16* __restrict__ w_router, int ldw) {
    const int r = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (r >= a.T) return;
    const float* h = a.h + (size_t)r * a.ldh;
    const bool vec = router_vec_ok(a.W, ldw, a.ldh);
    const int rows = a.E + a.n_extra;                     // (rows behind the experts': per-row scalars the feed-forward also needs)
    for (int e0 = 0; e0 < rows; e0 += 4) {
        float z[4];
        router_dots<4>(h, w_router + (size_t)e0 * ldw, ldw, a.W, min(4, rows - e0), lane, vec, z);
        if (lane < min(4, rows - e0)) a.router_logits[(size_t)r * a.ldr + e0 + lane] = lane == 0 ? z[0] : lane == 1 ? z[1] : lane == 2 ? z[2] : z[3];
    }
}

// Expert choice for one row by one warp.  z: the row's router logits; sc / ch / gs: 256 floats each of this warp's scratch.
// Scores = softmax over all experts or element-wise sigmoid; the choice value adds the selection bias; with n_groups > 1 only the
// experts of the `keep` groups with the largest (sum of the two largest choice values) stay eligible -- the others count as
// minus infinity; the `top` largest choice values win (ties: lowest index) and carry the plain scores as weights.
__device__ __forceinline__ void choose_experts(const MoeArgs& a, const float* z, int r, int lane, float* sc, float* ch, float* gs) {
    const int E = a.E;
    if (a.score_fn == 1) {
        for (int e = lane; e < E; e += 32) sc[e] = 1.f / (1.f + expf(-z[e]));
    } else {
        float mx = -INFINITY;
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
        mx = warp_max(mx);
        float den = 0.f;
        for (int e = lane; e < E; e += 32) den += expf(z[e] - mx);
        den = warp_sum(den);
        for (int e = lane; e < E; e += 32) sc[e] = expf(z[e] - mx) / den;
    }
    for (int e = lane; e < E; e += 32) ch[e] = sc[e] + (a.correction ? a.correction[e] : 0.f);
    __syncwarp();
    if (a.n_groups > 1) {
        const int per = E / a.n_groups;
        for (int g = lane; g < a.n_groups; g += 32) {
            float b0 = -INFINITY, b1 = -INFINITY;
            for (int i = 0; i < per; ++i) { const float v = ch[g * per + i]; if (v > b0) { b1 = b0; b0 = v; } else if (v > b1) b1 = v; }
            gs[g] = per > 1 ? b0 + b1 : b0;
        }
        __syncwarp();
        unsigned long long kept[4] = {0, 0, 0, 0};
        for (int k = 0; k < a.keep; ++k) {
            float bv = -INFINITY; int bi = 0x7fffffff;
            for (int g = lane; g < a.n_groups; g += 32)
                if (!((kept[g >> 6] >> (g & 63)) & 1ull) && gs[g] > bv) { bv = gs[g]; bi = g; }
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
            }
            if (bi == 0x7fffffff)                        // (no comparable value left: the lowest group not kept yet)
                for (int g = 0; g < a.n_groups; ++g) if (!((kept[g >> 6] >> (g & 63)) & 1ull)) { bi = g; break; }
            kept[bi >> 6] |= 1ull << (bi & 63);
        }
        for (int e = lane; e < E; e += 32) { const int g = e / per; if (!((kept[g >> 6] >> (g & 63)) & 1ull)) ch[e] = -INFINITY; }
        __syncwarp();
    }
    unsigned long long taken[4] = {0, 0, 0, 0};         // E <= 256: bit per expert, same in every lane
    for (int k = 0; k < a.top; ++k) {
        float bv = -INFINITY; int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32)
            if (!((taken[e >> 6] >> (e & 63)) & 1ull) && (ch[e] > bv)) { bv = ch[e]; bi = e; }
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (bi == 0x7fffffff) {                          // nothing eligible is left (every value minus infinity or NaN): lowest free index, weight 0
            for (int e = 0; e < E; ++e) if (!((taken[e >> 6] >> (e & 63)) & 1ull)) { bi = e; break; }
            if (lane == 0) { a.sel_e[(size_t)r * a.top + k] = bi; a.sel_w[(size_t)r * a.top + k] = 0.f; }
        } else if (lane == 0) { a.sel_e[(size_t)r * a.top + k] = bi; a.sel_w[(size_t)r * a.top + k] = sc[bi]; }
        taken[bi >> 6] |= 1ull << (bi & 63);
    }
}

// One warp per row, logits from global memory.
__global__ void __launch_bounds__(128) route_kernel(MoeArgs a) {
    __shared__ float scr[4][3][256];
    const int warp = threadIdx.x >> 5, r = blockIdx.x * 4 + warp, lane = threadIdx.x & 31;
    if (r >= a.T) return;
    choose_experts(a, a.router_logits + (size_t)r * a.ldr, r, lane, scr[warp][0], scr[warp][1], scr[warp][2]);
    if (a.n_extra > 0 && lane == 0) a.extra_out[r] = 1.f / (1.f + expf(-a.router_logits[(size_t)r * a.ldr + a.E]));
}

// Few rows (decode): router logits and the choice in one block per row.  Warp w computes the logits of experts w, w + 8, ...
// (f32 products of the f32 row with the bf16 router rows, lanes striding the width), warp 0 then selects as route_kernel does.
__global__ void __launch_bounds__(256) route_rows_kernel(MoeArgs a, const bf16* __restrict__ w_router, int ldw) {
    __shared__ float z[256 + 4];
    __shared__ float scr[3][256];
    const int r = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float* h = a.h + (size_t)r * a.ldh;
    const bool vec = router_vec_ok(a.W, ldw, a.ldh);
    for (int e = warp; e < a.E + a.n_extra; e += 8) {
        float acc;
        router_dots<1>(h, w_router + (size_t)e * ldw, ldw, a.W, 1, lane, vec, &acc);
        if (lane == 0) { z[e] = acc; a.router_logits[(size_t)r * a.ldr + e] = acc; }
    }
    __syncthreads();
    if (warp != 0) return;
    choose_experts(a, z, r, lane, scr[0], scr[1], scr[2]);
    if (a.n_extra > 0 && lane == 0) a.extra_out[r] = 1.f / (1.f + expf(-z[a.E]));
}

// Counting sort of the (row, choice) pairs by expert + the tile map of the grouped linears (32 pairs per tile).  One block.
__global__ void moe_sort_kernel(MoeArgs a) {
    extern __shared__ int sh[];
    int* cnt = sh; int* off = sh + a.E; int* fill = sh + 2 * a.E;
    const int n = a.T * a.top;
    for (int e = threadIdx.x; e < a.E; e += blockDim.x) { cnt[e] = 0; fill[e] = 0; }
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) atomicAdd(&cnt[a.sel_e[i]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int o = 0, t = 0;
        for (int e = 0; e < a.E; ++e) {
            off[e] = o;
            for (int r0 = 0; r0 < cnt[e]; r0 += 32) { a.tile_e[t] = e; a.tile_r0[t] = o + r0; a.tile_n[t] = min(32, cnt[e] - r0); ++t; }
            o += cnt[e];
        }
        *a.n_tiles = t;
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= a.E; e += blockDim.x) a.offs[e] = e < a.E ? off[e] : n;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int e = a.sel_e[i], at = off[e] + atomicAdd(&fill[e], 1);
        a.sorted[at] = i;
        a.inv[i] = at;
    }
}

// Grouped linear: tile = 32 pairs of one expert x 64 output columns.  UP: act[pair] = gelu_erf(up_e h[row of pair]); else y[pair] = down_e act[pair].
template <bool UP>
__global__ void __launch_bounds__(256) moe_linear_kernel(MoeArgs a) {
    __shared__ float sa[16][32 + 1], sw[16][64 + 4];
    __shared__ int spair[32];
    const int tile = blockIdx.y;
    if (tile >= *a.n_tiles) return;
    const int e = a.tile_e[tile], r0 = a.tile_r0[tile], nr = a.tile_n[tile];
    const int N = UP ? (a.gated ? 2 * a.F : a.F) : a.W, K = UP ? a.W : a.F, ldw = UP ? a.ldwu : a.ldwd;
    const bf16* Wt = UP ? a.up[e] : a.down[e];
    const int n0 = blockIdx.x * 64, tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;      // thread: 2 pairs x 4 columns
    if (tid < 32) spair[tid] = tid < nr ? a.sorted[r0 + tid] : -1;
    __syncthreads();
    float acc[2][4] = {};
    for (int k0 = 0; k0 < K; k0 += 16) {
        for (int i = tid; i < 32 * 16; i += 256) {
            const int r = i >> 4, k = i & 15, pr = spair[r];
            float v = 0.f;
            if (pr >= 0 && k0 + k < K) v = UP ? a.h[(size_t)(pr / a.top) * a.ldh + k0 + k] : a.act[(size_t)pr * a.lda + k0 + k];
            sa[k][r] = v;
        }
        for (int i = tid; i < 64 * 16; i += 256) {
            const int r = i >> 4, k = i & 15;
            sw[k][r] = (n0 + r < N && k0 + k < K) ? __bfloat162float(Wt[(size_t)(n0 + r) * ldw + k0 + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            const float a0 = sa[k][ty * 2], a1 = sa[k][ty * 2 + 1];
#pragma unroll
            for (int j = 0; j < 4; ++j) { const float w = sw[k][tx * 4 + j]; acc[0][j] = fmaf(a0, w, acc[0][j]); acc[1][j] = fmaf(a1, w, acc[1][j]); }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int pr = spair[ty * 2 + i];
        if (pr < 0) continue;
        const float ws = (UP && a.scale_input) ? a.sel_w[pr] : 1.f;      // the expert reads weight * h: its first products are linear in h
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            if (UP) {
                if (!a.gated) a.act[(size_t)pr * a.lda + n] = gelu_erf_f(acc[i][j] * ws);
                else if (!(j & 1)) a.act[(size_t)pr * a.lda + (n >> 1)] = glu_pair_f(acc[i][j] * ws, acc[i][j + 1] * ws, a.glu_limit);      // columns (2m, 2m + 1) = (gate_m, up_m)
            } else a.y[(size_t)pr * a.ldy + n] = acc[i][j];
        }
    }
}

// x[r] += sum over the row's choices, in choice order, of weight * expert output (y rows by pair, or by place in the sorted list);
// the weight is 1 where it already multiplied the expert's input.  Optionally, before the add: an every-token expert's output times a
// per-row scalar joins the sum, a per-column scale applies, and a sigmoid gate per element multiplies the whole.
__global__ void moe_combine_kernel(MoeArgs a, int y_sorted) {
    const int r = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= a.W) return;
    float s = 0.f;
    for (int k = 0; k < a.top; ++k) {
        const int pr = r * a.top + k, row = y_sorted ? a.inv[pr] : pr;
        s = a.scale_input ? s + a.y[(size_t)row * a.ldy + c] : fmaf(a.sel_w[pr], a.y[(size_t)row * a.ldy + c], s);
    }
    if (a.shared_y) s = fmaf(a.shared_w ? a.shared_w[r] : 1.f, a.shared_y[(size_t)r * a.lds + c], s);
    if (a.out_scale) s *= a.out_scale[c];
    if (a.gate) s *= 1.f / (1.f + expf(-(a.gate[(size_t)r * a.ldg + c] + (a.gate_bias ? a.gate_bias[c] : 0.f))));
    a.x[(size_t)r * a.ldx + c] += s;
}
__global__ void moe_gather_kernel(MoeArgs a, ActOut src, ActOut dst) {
    const int i = blockIdx.x, r = a.sorted[i] / a.top;
    if (a.scale_input) {                                    // the expert's input is weight * h, rounded as the planes round it
        const float ws = a.sel_w[a.sorted[i]];
        const bf16* sh = src.hi + (size_t)r * src.ldb;
        bf16* dh = dst.hi + (size_t)i * dst.ldb;
        for (int c = threadIdx.x; c < src.ldb; c += blockDim.x) {
            const float v = (__bfloat162float(sh[c]) + (src.lo_off ? __bfloat162float(sh[c + src.lo_off]) : 0.f)) * ws;
            const bf16 h = __float2bfloat16_rn(v);
            dh[c] = h;
            if (dst.lo_off) dh[c + dst.lo_off] = __float2bfloat16_rn(v - __bfloat162float(h));
        }
        return;
    }
    const uint4* s = reinterpret_cast<const uint4*>(src.hi + (size_t)r * src.ldb);
    uint4* d = reinterpret_cast<uint4*>(dst.hi + (size_t)i * dst.ldb);
    const int n = src.ldb / 8;                              // padded widths: multiples of 8 elements
    for (int c = threadIdx.x; c < n; c += blockDim.x) d[c] = s[c];
    if (src.lo_off && dst.lo_off) {
        const uint4* sl = reinterpret_cast<const uint4*>(src.hi + src.lo_off + (size_t)r * src.ldb);
        uint4* dl = reinterpret_cast<uint4*>(dst.hi + dst.lo_off + (size_t)i * dst.ldb);
        for (int c = threadIdx.x; c < n; c += blockDim.x) dl[c] = sl[c];
    }
}

constexpr int ARGMAX_PARTS = 64;
__device__ __forceinline__ void argmax_merge(float& bv, int& bi, float ov, int oi) { if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; } }
__global__ void __launch_bounds__(256) argmax_parts_kernel(const float* __restrict__ logits, int V, float* __restrict__ pv, int* __restrict__ pi) {
    __shared__ float sv[8];
    __shared__ int si[8];
    const int e = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float* row = logits + (size_t)e * V;
    const int per = (V + ARGMAX_PARTS - 1) / ARGMAX_PARTS, lo = blockIdx.x * per, hi = min(V, lo + per);
    float bv = -INFINITY; int bi = 0x7fffffff;
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) argmax_merge(bv, bi, row[i], i);
    for (int o = 16; o > 0; o >>= 1) argmax_merge(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
    if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w) argmax_merge(bv, bi, sv[w], si[w]);
        pv[e * ARGMAX_PARTS + blockIdx.x] = bv; pi[e * ARGMAX_PARTS + blockIdx.x] = bi;
    }
}
// one warp per row finishes the argmax (lowest index among maxima), feeds the token back and moves the positions on
__global__ void greedy_advance_kernel(const float* __restrict__ pv, const int* __restrict__ pi, int E, int* ids, int* row_pos, int* ent_pos0,
                                      uint32_t* out, int out_stride, int* step) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int t = *step;
    for (int e = warp; e < E; e += nw) {
        float bv = -INFINITY; int bi = 0x7fffffff;
        for (int i = lane; i < ARGMAX_PARTS; i += 32) argmax_merge(bv, bi, pv[e * ARGMAX_PARTS + i], pi[e * ARGMAX_PARTS + i]);
        for (int o = 16; o > 0; o >>= 1) argmax_merge(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
        if (lane == 0) {
            if (bi == 0x7fffffff) bi = 0;
            out[(size_t)e * out_stride + t] = (uint32_t)bi;
            ids[e] = bi; row_pos[e] += 1; ent_pos0[e] += 1;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) *step = t + 1;
}

// Experts for a handful of (row, expert) pairs -- a decode step: block = (16 output rows, pair); the pair's input vector sits in
// shared memory and every warp streams two weight rows with 16-byte loads (padded row widths are multiples of 256).
template <bool UP>
__global__ void __launch_bounds__(256) moe_gemv_kernel(MoeArgs a) {
    extern __shared__ float xs[];
    const int pr = blockIdx.y, e = a.sel_e[pr], lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int N = UP ? a.F : a.W, K = UP ? a.W : a.F, ldw = UP ? a.ldwu : a.ldwd;
    const float* x = UP ? a.h + (size_t)(pr / a.top) * a.ldh : a.act + (size_t)pr * a.lda;
    for (int k = threadIdx.x; k < ldw; k += blockDim.x) xs[k] = k < K ? x[k] : 0.f;
    __syncthreads();
    const bf16* Wt = UP ? a.up[e] : a.down[e];
    float pair[2] = {0.f, 0.f};
    for (int rr = 0; rr < 2; ++rr) {
        const int n = blockIdx.x * 16 + warp * 2 + rr;
        if (n >= (UP && a.gated ? 2 * N : N)) continue;
        const uint4* w8 = reinterpret_cast<const uint4*>(Wt + (size_t)n * ldw);
        float acc = 0.f;
        for (int k = lane; k < ldw / 8; k += 32) {
            const uint4 ww = ldg_stream(w8 + k);
            const float* xx = xs + 8 * k;
            acc = fmaf(bf16lo(ww.x), xx[0], acc); acc = fmaf(bf16hi(ww.x), xx[1], acc); acc = fmaf(bf16lo(ww.y), xx[2], acc); acc = fmaf(bf16hi(ww.y), xx[3], acc);
            acc = fmaf(bf16lo(ww.z), xx[4], acc); acc = fmaf(bf16hi(ww.z), xx[5], acc); acc = fmaf(bf16lo(ww.w), xx[6], acc); acc = fmaf(bf16hi(ww.w), xx[7], acc);
        }
        acc = warp_sum(acc);
        if (UP && a.scale_input) acc *= a.sel_w[pr];
        pair[rr] = acc;
        if (lane == 0) {
            if (UP) { if (!a.gated) a.act[(size_t)pr * a.lda + n] = gelu_erf_f(acc); }
            else a.y[(size_t)pr * a.ldy + n] = acc;
        }
    }
    // gated experts: the warp's two rows are (gate_m, up_m), m = blockIdx.x * 8 + warp
    if (UP && a.gated && lane == 0) {
        const int m = blockIdx.x * 8 + warp;
        if (m < N) a.act[(size_t)pr * a.lda + m] = glu_pair_f(pair[0], pair[1], a.glu_limit);
    }
}

inline int last_err() { return (int)cudaGetLastError(); }

}  // namespace

// ---------------------------------------------------------------------------------------------------------------- launchers
int embed_scale_rows_launch(cudaStream_t st, const int* ids, int T, const bf16* embed, int W, float scale, float* x, int ldx) {
    embed_scale_rows_kernel<<<T, 128, 0, st>>>(ids, T, embed, W, scale, x, ldx);
    return last_err();
}
int embed_sinpos_rows_launch(cudaStream_t st, const int* ids, const int* row_pos, int T, const bf16* embed, int W, const float* freq, float* x, int ldx) {
    embed_sinpos_rows_kernel<<<T, 128, 0, st>>>(ids, row_pos, embed, W, freq, x, ldx);
    return last_err();
}
int post_norm_add_launch(cudaStream_t st, const float* y1, int ld1, const float* b1, const float* w1, const float* y2, int ld2, const float* w2,
                         const float* norm_w, float eps, float* x, int ldx, int T, int W, const ActOut& planes) {
    if (!y1 || !norm_w || planes.f) return -1000;
    post_norm_add_kernel<<<T, 256, 0, st>>>(y1, ld1, b1, w1, y2, ld2, w2, norm_w, eps, x, ldx, W, planes);
    return last_err();
}
int dyt_rows_launch(cudaStream_t st, const float* x, int ldx, const int* rows, int R, int W, const float* alpha, const float* w, const float* b,
                    const ActOut& out) {
    dyt_rows_kernel<<<R, 128, 0, st>>>(x, ldx, rows, W, alpha, w, b, out);
    return last_err();
}
int greedy_advance_launch(cudaStream_t st, const float* logits, int V, int E, float* part_val, int* part_idx, int* ids, int* row_pos,
                          int* ent_pos0, uint32_t* out, int out_stride, int* step) {
    argmax_parts_kernel<<<dim3(ARGMAX_PARTS, E), 256, 0, st>>>(logits, V, part_val, part_idx);
    int e = last_err();
    if (e) return e;
    greedy_advance_kernel<<<1, 256, 0, st>>>(part_val, part_idx, E, ids, row_pos, ent_pos0, out, out_stride, step);
    return last_err();
}
int gather_rows_launch(cudaStream_t st, const float* src, int lds, const int* rows, int R, int W, float* dst, int ldd) {
    gather_rows_kernel<<<R, 128, 0, st>>>(src, lds, rows, W, dst, ldd);
    return last_err();
}
int linear_f32_launch(cudaStream_t st, const float* A, int lda, const bf16* W, int ldw, int M, int N, int K, int mode, float* C, int ldc,
                      const float* col_scale, const float* gate, int ldg, const float* gate_bias) {
    if (M <= 0 || N <= 0 || K <= 0) return -1000;
    const dim3 grid((N + 63) / 64, (M + 63) / 64);
    if (mode == LIN_RESID) linear_f32_kernel<LIN_RESID><<<grid, 256, 0, st>>>(A, lda, W, ldw, M, N, K, C, ldc, col_scale, gate, ldg, gate_bias);
    else linear_f32_kernel<LIN_STORE><<<grid, 256, 0, st>>>(A, lda, W, ldw, M, N, K, C, ldc, nullptr, nullptr, 0, nullptr);
    return last_err();
}
int rms_rows_launch(cudaStream_t st, const float* x, int ldx, const int* rows, int R, int W, float eps, const float* w1, const ActOut& out1,
                    const float* w2, const ActOut& out2, int groups) {
    if (groups < 1 || W % groups) return -1000;
    rms_rows_kernel<<<R, 256, 0, st>>>(x, ldx, rows, W, eps, w1, out1, w2, out2, groups);
    return last_err();
}
int store_rows_launch(cudaStream_t st, const float* src, int lds, int T, int W, const ActOut& dst, int col0) {
    store_rows_kernel<<<T, 128, 0, st>>>(src, lds, W, dst, col0);
    return last_err();
}
int silu_glu_launch(cudaStream_t st, const float* gu, int ld, int T, int F, const ActOut& out, float limit) {
    silu_glu_kernel<<<dim3((F + 127) / 128, T), 128, 0, st>>>(gu, ld, F, out, limit);
    return last_err();
}
int attn_prep_launch(cudaStream_t st, const RaggedBatch& rb, const AttnPrepArgs& a) {
    if (a.rot_dims < 0 || (a.rot_dims & 1) || a.rot_dims > a.d || a.rot_dims > 4096) return -1000;
    if (a.v_from_k && a.d != a.dv) return -1000;
    const size_t sm = (size_t)a.rot_dims * sizeof(float);
    if (a.kv_f32) attn_prep_kernel<float><<<rb.T, 256, sm, st>>>(rb, a);
    else attn_prep_kernel<bf16><<<rb.T, 256, sm, st>>>(rb, a);
    return last_err();
}
template <typename KT, int REP>
static int sink_attention_launch_t(cudaStream_t st, const RaggedBatch& rb, const SinkAttnArgs& a) {
    const int rep = a.H / a.G, nb = (rep + REP - 1) / REP;
    size_t smem = (size_t)(REP * a.d + 2 * ATT_WARPS * REP + ATT_WARPS * REP * a.dv) * sizeof(float);
    if (smem > 200 * 1024) return -1000;
    // per-warp staging patches for the key / value tiles where the widths allow 16-byte copies and the patches fit
    const int planes = (sizeof(KT) == 2 && a.kv_lo_off) ? 2 : 1;
    const size_t patch = (size_t)ATT_WARPS * 32 * planes * ((size_t)a.d * sizeof(KT) + 16 + (a.kv_shared ? 0 : (size_t)a.dv * sizeof(KT) + 16)) + 16;
    // ... and the launch is small (a decode step: about two blocks per SM at most).  A launch of thousands of blocks hides its load
    // latency by residency instead, which the patches' shared memory would take away.
    const int stage = ((a.d & 7) == 0 && (a.dv & 7) == 0 && smem + patch <= 200 * 1024 && (long long)rb.T * a.G * nb * a.nsplit <= 300) ? 1 : 0;
    if (stage) smem += patch;
    static SmemOptIn seen, seen_staged;
    if (stage) {
        if (const int e = ensure_dyn_smem(sink_attention_kernel<KT, REP, true>, smem, seen_staged)) return e;
        sink_attention_kernel<KT, REP, true><<<dim3(rb.T, a.G * nb, a.nsplit), ATT_WARPS * 32, smem, st>>>(rb, a);
        return last_err();
    }
    if (const int e = ensure_dyn_smem(sink_attention_kernel<KT, REP, false>, smem, seen)) return e;
    sink_attention_kernel<KT, REP, false><<<dim3(rb.T, a.G * nb, a.nsplit), ATT_WARPS * 32, smem, st>>>(rb, a);
    return last_err();
}
template <typename KT>
static int sink_attention_launch_k(cudaStream_t st, const RaggedBatch& rb, const SinkAttnArgs& a) {
    const int rep = a.H / a.G;
    // few blocks (a decode step): one query head per block keeps more SMs busy than sharing the keys would save
    if (rep == 1 || (long long)rb.T * a.H * a.nsplit <= 1024) return sink_attention_launch_t<KT, 1>(st, rb, a);
    if (rep == 2) return sink_attention_launch_t<KT, 2>(st, rb, a);
    if (rep <= 4) return sink_attention_launch_t<KT, 4>(st, rb, a);
    return sink_attention_launch_t<KT, 8>(st, rb, a);
}
int sink_attention_launch(cudaStream_t st, const RaggedBatch& rb, const SinkAttnArgs& a) {
    if (a.dv > 32 * ATT_MAXC || a.H % a.G) return -1000;
    if (a.kv_shared && (a.k_pool != a.v_pool || a.d != a.dv)) return -1000;
    int e = a.kv_f32 ? sink_attention_launch_k<float>(st, rb, a) : sink_attention_launch_k<bf16>(st, rb, a);
    if (e || a.nsplit == 1) return e;
    if (a.nsplit > 64) return -1000;
    sink_attention_merge_kernel<<<dim3(rb.T, a.H), 128, 0, st>>>(a);
    return last_err();
}
int mamba2_launch_count(bool single_rows, int max_len) { return single_rows ? 3 : max_len >= SSD_SEG_MIN ? 6 : 4; }
size_t mamba2_seg_floats(int entries, int heads, int N, int P) { return (size_t)entries * SSD_SEGS * heads * ((size_t)N * P + 1); }
size_t mamba2_seg_decay_offset(int entries, int heads, int N, int P) { return (size_t)entries * SSD_SEGS * heads * (size_t)N * P; }
int mamba2_mixer_launch(cudaStream_t st, const RaggedBatch& rb, const Mamba2Args& a) {
    const int inner = a.heads * a.P, C = inner + 2 * a.groups * a.N;
    if (a.N > SSD_NS * SSD_MAXR || a.heads % a.groups || inner % a.norm_groups || a.taps < 1) return -1000;
    int e;
    if (a.single_rows) {
        conv_step_kernel<<<dim3((C + 127) / 128, rb.E), 128, 0, st>>>(rb, a, C, inner);
        if ((e = last_err())) return e;
    } else {
        conv_silu_kernel<<<dim3((C + 127) / 128, rb.T), 128, 0, st>>>(rb, a, C, inner);
        if ((e = last_err())) return e;
        if (a.taps > 1) {
            conv_window_kernel<<<dim3((C + 127) / 128, rb.E), 128, 0, st>>>(rb, a, C, inner);
            if ((e = last_err())) return e;
        }
    }
    const dim3 sgrid(rb.E, a.heads, (a.P + SSD_COLS - 1) / SSD_COLS);
    const int nr = (a.N + SSD_NS - 1) / SSD_NS, sthreads = SSD_COLS * SSD_NS;
    const int rr = nr <= 4 ? 4 : nr <= 8 ? 8 : nr <= 16 ? 16 : 32;
    const size_t ssm = (size_t)(2 * SSD_CH * (SSD_COLS + 2 * ssd_npad(a.N, rr) + 4) + 2 * SSD_CH) * sizeof(float);      // <= 78 KB at N = 256
    const bool segs = a.seg_state != nullptr && a.max_len >= SSD_SEG_MIN;
    auto run = [&](auto kern, SmemOptIn& seen, dim3 grid) -> int {
        if (const int er = ensure_dyn_smem(kern, ssm, seen)) return er;
        kern<<<grid, sthreads, ssm, st>>>(rb, a, C);
        return last_err();
    };
    auto scan = [&](auto k4, auto k8, auto k16, auto k32, SmemOptIn* seen, dim3 grid) -> int {
        return nr <= 4 ? run(k4, seen[0], grid) : nr <= 8 ? run(k8, seen[1], grid) : nr <= 16 ? run(k16, seen[2], grid) : run(k32, seen[3], grid);
    };
    static SmemOptIn seen0[4], seen1[4], seen2[4];
    if (!segs) {
        if ((e = scan(ssd_scan_kernel<4, 0>, ssd_scan_kernel<8, 0>, ssd_scan_kernel<16, 0>, ssd_scan_kernel<32, 0>, seen0, sgrid))) return e;
    } else {
        const dim3 ggrid(rb.E * SSD_SEGS, a.heads, sgrid.z);
        if ((e = scan(ssd_scan_kernel<4, 1>, ssd_scan_kernel<8, 1>, ssd_scan_kernel<16, 1>, ssd_scan_kernel<32, 1>, seen1, ggrid))) return e;
        ssd_seg_prefix_kernel<<<dim3(rb.E, a.heads, 8), 256, 0, st>>>(rb, a);
        if ((e = last_err())) return e;
        if ((e = scan(ssd_scan_kernel<4, 2>, ssd_scan_kernel<8, 2>, ssd_scan_kernel<16, 2>, ssd_scan_kernel<32, 2>, seen2, ggrid))) return e;
    }
    if ((e = last_err())) return e;
    gated_group_rms_kernel<<<dim3(rb.T, a.norm_groups), 128, 0, st>>>(a);
    return last_err();
}
int clamped_glu_launch(cudaStream_t st, const float* gu, int ld, int stride, int up_off, int T, int F, float limit, const ActOut& out) {
    clamped_glu_kernel<<<dim3((F + 127) / 128, T), 128, 0, st>>>(gu, ld, stride, up_off, F, limit, out);
    return last_err();
}
static bool moe_few_pairs(const MoeArgs& a) {
    return a.T * a.top <= 32 && (a.ldwu & 255) == 0 && (a.ldwd & 255) == 0 && (size_t)std::max(a.ldwu, a.ldwd) * 4 <= 48 * 1024;
}
int moe_route_launch(cudaStream_t st, const MoeArgs& a, const bf16* w_router, int ldw) {
    if (a.E > 256 || a.top > a.E || a.top < 1) return -1000;
    if (a.n_groups > 1 && (a.E % a.n_groups || a.keep < 1 || a.keep > a.n_groups || a.top > a.keep * (a.E / a.n_groups))) return -1000;
    int e;
    if (a.T <= 64) {          // few rows: logits + selection in one launch
        route_rows_kernel<<<a.T, 256, 0, st>>>(a, w_router, ldw);
        e = last_err();
    } else {
        router_logits_kernel<<<(a.T + 7) / 8, 256, 0, st>>>(a, w_router, ldw);
        if ((e = last_err())) return e;
        route_kernel<<<(a.T + 3) / 4, 128, 0, st>>>(a);
        e = last_err();
    }
    if (e || moe_few_pairs(a)) return e;                  // (a handful of pairs go through moe_gemv, which reads the choices as they are)
    moe_sort_kernel<<<1, 1024, (size_t)3 * a.E * sizeof(int), st>>>(a);
    return last_err();
}
int moe_experts_launch(cudaStream_t st, const MoeArgs& a) {
    if (moe_few_pairs(a)) {
        moe_gemv_kernel<true><<<dim3(((a.gated ? 2 * a.F : a.F) + 15) / 16, a.T * a.top), 256, (size_t)a.ldwu * 4, st>>>(a);
        int e = last_err();
        if (e) return e;
        moe_gemv_kernel<false><<<dim3((a.W + 15) / 16, a.T * a.top), 256, (size_t)a.ldwd * 4, st>>>(a);
        if ((e = last_err())) return e;
        return moe_combine_launch(st, a, false);
    }
    moe_linear_kernel<true><<<dim3(((a.gated ? 2 * a.F : a.F) + 63) / 64, a.max_tiles), 256, 0, st>>>(a);
    int e = last_err();
    if (e) return e;
    moe_linear_kernel<false><<<dim3((a.W + 63) / 64, a.max_tiles), 256, 0, st>>>(a);
    if ((e = last_err())) return e;
    return moe_combine_launch(st, a, false);
}
int moe_gather_launch(cudaStream_t st, const MoeArgs& a, const ActOut& src, const ActOut& dst) {
    if (!src.hi || !dst.hi || src.ldb != dst.ldb || (src.ldb & 7)) return -1000;
    moe_gather_kernel<<<a.T * a.top, 128, 0, st>>>(a, src, dst);
    return last_err();
}
int moe_combine_launch(cudaStream_t st, const MoeArgs& a, bool y_sorted) {
    moe_combine_kernel<<<dim3((a.W + 127) / 128, a.T), 128, 0, st>>>(a, y_sorted ? 1 : 0);
    return last_err();
}

}  // namespace cb
