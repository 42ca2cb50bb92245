// Recurrent mixers of ragged-batch steps whose state is carried per sequence slot in f32 (see ragged.cuh):
//   * the selective scan with a state per channel (Mamba-1): decay exp(dt_c A[c, n]) per channel and state entry;
//   * the matrix memory with exponential gates and a running maximum (mLSTM): a scalar decay per head and token.
// Both walk a portion token by token; a thread keeps its share of the state in registers for the whole portion, the step inputs of
// SC_CH tokens at a time are staged in shared memory (cp.async, double-buffered), and everything that enters the recurrence (step
// sizes, softplus, decays, gates, the running maximum) is computed in f32.  A row's result depends on its own sequence only: the
// split of the state over lanes and the order of the lane sums are launch constants.
#include "ragged.cuh"
#include "ragged_dev.cuh"

#include <algorithm>
#include <type_traits>

namespace cb {

namespace {

constexpr int SC_NS = 8;        // lanes that share one channel (Mamba-1) / one value column (mLSTM): each owns a contiguous slice of the state
constexpr int SC_COLS = 16;     // channels / value columns per block -> 128 threads
constexpr int SC_CH = 16;       // tokens staged per chunk
// A long portion is cut into SC_SEGS segments that run side by side (a scan has one resident warp per scheduler and waits on its
// own dependent chain most of the time).  Both recurrences are linear in the state with a decay that does not depend on it, so
//   S_end(segment) = (product of the segment's decays) * S_start + S_local(segment run from zero),
// element by element.  MODE 1 runs every segment but the last from zero and leaves S_local and what the decay product needs;
// a prefix kernel turns them into each segment's start state; MODE 2 is the scan proper from those start states (the last segment
// leaves the sequence's new state).  MODE 0 = one segment, everything.
constexpr int SC_SEGS = 8, SC_SEG_MIN = 512;          // segmented from this many rows in the step's longest entry
__host__ __device__ inline int sc_seg_len(int len) { return ((len + SC_SEGS - 1) / SC_SEGS + SC_CH - 1) / SC_CH * SC_CH; }

inline int last_err() { return (int)cudaGetLastError(); }

__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float log_sigmoid_f(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

// ---------------------------------------------------------------------------------------------------------------- Mamba-1
// Staged layout of a state vector of n entries cut into eight runs of R (one per lane of a channel): from R = 4 on every run is
// followed by 4 pad floats, which spreads the eight runs of a warp over all banks and lets a lane read its run as float4.
__host__ __device__ inline int sc_idx(int n, int R) { return R >= 4 ? n + 4 * (n / R) : n; }
__host__ __device__ inline int sc_pad(int R) { return R >= 4 ? SC_NS * (R + 4) : SC_NS * R; }

// Step sizes, block = (DT_TOK tokens, 128 channels): dt[t, c] = softplus(sum_k w_dt[c, k] low[t, k] + b[c]), k in order, f32.
// w_dtT is the projection transposed, [dt_rank, inner]: a warp's channels read it side by side.
template <int DT_TOK>
__global__ void __launch_bounds__(128) mamba1_dt_kernel(Mamba1Args a, int T) {
    extern __shared__ __align__(16) float slow[];             // [DT_TOK][dt_rank]
    const int t0 = blockIdx.x * DT_TOK, c = blockIdx.y * 128 + threadIdx.x, Rk = a.dt_rank, nt = min(DT_TOK, T - t0);
    for (int i = threadIdx.x; i < DT_TOK * Rk; i += 128) slow[i] = i / Rk < nt ? a.low[(size_t)(t0 + i / Rk) * a.ldl + i % Rk] : 0.f;
    __syncthreads();
    if (c >= a.inner) return;
    float acc[DT_TOK];
#pragma unroll
    for (int t = 0; t < DT_TOK; ++t) acc[t] = 0.f;
    const float* wc = a.w_dtT + c;
    int k = 0;
    for (; k + 8 <= Rk; k += 8) {                             // eight weights requested before the first is used
        float w[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) w[u] = wc[(size_t)(k + u) * a.inner];
#pragma unroll
        for (int u = 0; u < 8; ++u)
#pragma unroll
            for (int t = 0; t < DT_TOK; ++t) acc[t] = fmaf(w[u], slow[t * Rk + k + u], acc[t]);
    }
    for (; k < Rk; ++k) {
        const float w = wc[(size_t)k * a.inner];
#pragma unroll
        for (int t = 0; t < DT_TOK; ++t) acc[t] = fmaf(w, slow[t * Rk + k], acc[t]);
    }
    const float b = a.dt_b[c];
#pragma unroll
    for (int t = 0; t < DT_TOK; ++t) if (t < nt) a.dt[(size_t)(t0 + t) * a.lddt + c] = softplus_f(acc[t] + b);
}

// Block = (entry, SC_COLS channels); thread (cl, ns) owns the state entries n = ns * R .. ns * R + R - 1 of channel c0 + cl in
// registers for the whole portion.  The recurrence is one multiply-add deep per token; what would serialise it is the operand
// fetch, so the step inputs of SC_CH tokens at a time (u, dt, z of the block's channels; B and C) are staged in shared memory with
// cp.async, double-buffered: chunk c + 1 is in flight while chunk c is consumed.  A chunk's outputs wait in shared memory and leave
// together, gated by silu(z).
template <int R, int MODE>
__global__ void __launch_bounds__(SC_COLS * SC_NS) mamba1_scan_kernel(RaggedBatch rb, Mamba1Args a) {
    extern __shared__ __align__(16) float sm[];
    const int e = MODE == 0 ? blockIdx.x : blockIdx.x / SC_SEGS, seg = MODE == 0 ? 0 : blockIdx.x % SC_SEGS, c0 = blockIdx.y * SC_COLS;
    const int ns = threadIdx.x & (SC_NS - 1), cl = threadIdx.x / SC_NS, c = c0 + cl;
    const int N = a.N, NP = sc_pad(R), PT = 3 * SC_COLS + 2 * NP;       // per staged token: u | dt | z | B | C
    const bool live = c < a.inner;
    const int full_len = rb.ent_len[e], slot = rb.ent_slot[e];
    const int seg_len = MODE == 0 ? full_len : sc_seg_len(full_len), seg0 = seg * seg_len;
    if (seg0 >= full_len) return;                             // (a short entry has fewer segments)
    const bool last_seg = seg0 + seg_len >= full_len;
    if (MODE == 1 && last_seg) return;                        // nothing follows the last segment: its end state is MODE 2's to leave
    const int len = min(seg_len, full_len - seg0), r0 = rb.ent_row0[e] + seg0;
    float* stage[2] = {sm, sm + SC_CH * PT};
    float* sy = sm + 2 * SC_CH * PT;                                    // [CH][COLS]
    const int n0 = ns * R, ncol = min(SC_COLS, a.inner - c0);
    for (int i = threadIdx.x; i < 2 * SC_CH * PT; i += blockDim.x) sm[i] = 0.f;       // entries past N, channels past the last stay zero
    float s[R], An[R];
    float* S = a.state + ((size_t)slot * a.inner + (live ? c : 0)) * N;
    float* Sg = MODE == 0 ? S : a.seg_state + (((size_t)e * SC_SEGS + seg) * a.inner + (live ? c : 0)) * N;      // MODE 1 leaves S_local here, MODE 2 starts from it
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const bool ok = live && n0 + i < N;
        s[i] = (ok && MODE != 1) ? Sg[n0 + i] : 0.f;
        An[i] = ok ? a.A[(size_t)c * N + n0 + i] : 0.f;
    }
    float dt_sum = 0.f;                                       // MODE 1: the segment's decay product is exp(A * sum of its step sizes)
    const float Dc = live ? a.D[c] : 0.f;
    __syncthreads();
    // 16-byte copies when every piece starts on a 16-byte boundary (the usual geometry), 4-byte copies otherwise
    const bool wide = ((N | a.dt_rank | a.inner | a.ldu | a.ldl | a.ldz | a.lddt) & 3) == 0 && (R >= 4 ? (R & 3) == 0 : true) && ncol == SC_COLS &&
                      (((size_t)a.u | (size_t)a.low | (size_t)a.z | (size_t)a.dt) & 15) == 0;
    auto fetch = [&](int ch, float* dst) {
        const int t0 = ch * SC_CH, nt = min(SC_CH, len - t0);
        if (wide) {
            const int nq = N >> 2, per = 12 + 2 * nq;
            for (int i = threadIdx.x; i < nt * per; i += blockDim.x) {
                const int t = i / per, k = i - t * per, r = r0 + t0 + t;
                float* d0 = dst + t * PT;
                if (k < 4) cp_async16s(d0 + 4 * k, a.u + (size_t)r * a.ldu + c0 + 4 * k);
                else if (k < 8) cp_async16s(d0 + SC_COLS + 4 * (k - 4), a.dt + (size_t)r * a.lddt + c0 + 4 * (k - 4));
                else if (k < 12) cp_async16s(d0 + 2 * SC_COLS + 4 * (k - 8), a.z + (size_t)r * a.ldz + c0 + 4 * (k - 8));
                else if (k < 12 + nq) { const int n = 4 * (k - 12); cp_async16s(d0 + 3 * SC_COLS + sc_idx(n, R), a.low + (size_t)r * a.ldl + a.dt_rank + n); }
                else { const int n = 4 * (k - 12 - nq); cp_async16s(d0 + 3 * SC_COLS + NP + sc_idx(n, R), a.low + (size_t)r * a.ldl + a.dt_rank + N + n); }
            }
        } else {
            const int per = 3 * SC_COLS + 2 * N;
            for (int i = threadIdx.x; i < nt * per; i += blockDim.x) {
                const int t = i / per, k = i - t * per, r = r0 + t0 + t;
                float* d0 = dst + t * PT;
                if (k < 3 * SC_COLS) {
                    const int which = k / SC_COLS, cc = k % SC_COLS;
                    if (cc >= ncol) continue;
                    const float* src = which == 0 ? a.u + (size_t)r * a.ldu : which == 1 ? a.dt + (size_t)r * a.lddt : a.z + (size_t)r * a.ldz;
                    cp_async4(d0 + k, src + c0 + cc);
                } else if (k < 3 * SC_COLS + N) { const int n = k - 3 * SC_COLS; cp_async4(d0 + 3 * SC_COLS + sc_idx(n, R), a.low + (size_t)r * a.ldl + a.dt_rank + n); }
                else { const int n = k - 3 * SC_COLS - N; cp_async4(d0 + 3 * SC_COLS + NP + sc_idx(n, R), a.low + (size_t)r * a.ldl + a.dt_rank + N + n); }
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const int nch = (len + SC_CH - 1) / SC_CH;
    fetch(0, stage[0]);
    for (int ch = 0; ch < nch; ++ch) {
        if (ch + 1 < nch) { fetch(ch + 1, stage[(ch + 1) & 1]); asm volatile("cp.async.wait_group 1;" ::: "memory"); }
        else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        const float* st = stage[ch & 1];
        const int nt = min(SC_CH, len - ch * SC_CH);
        const int tmax = (nt + 3) & ~3;                       // whole groups of four: a token past the end leaves the state as it is
#pragma unroll 4
        for (int t = 0; t < tmax; ++t) {
            const float* tk = st + t * PT;
            const float uv = tk[cl], dt = t < nt ? tk[SC_COLS + cl] : 0.f, dx = dt * uv;
            const float* Bt = tk + 3 * SC_COLS + sc_idx(n0, R);
            const float* Ct = Bt + NP;
            float y = 0.f;
            if constexpr ((R & 3) == 0) {
#pragma unroll
                for (int i = 0; i < R / 4; ++i) {
                    const float4 b = reinterpret_cast<const float4*>(Bt)[i], cc = reinterpret_cast<const float4*>(Ct)[i];
                    s[4 * i] = fmaf(__expf(dt * An[4 * i]), s[4 * i], dx * b.x); y = fmaf(s[4 * i], cc.x, y);
                    s[4 * i + 1] = fmaf(__expf(dt * An[4 * i + 1]), s[4 * i + 1], dx * b.y); y = fmaf(s[4 * i + 1], cc.y, y);
                    s[4 * i + 2] = fmaf(__expf(dt * An[4 * i + 2]), s[4 * i + 2], dx * b.z); y = fmaf(s[4 * i + 2], cc.z, y);
                    s[4 * i + 3] = fmaf(__expf(dt * An[4 * i + 3]), s[4 * i + 3], dx * b.w); y = fmaf(s[4 * i + 3], cc.w, y);
                }
            } else {
#pragma unroll
                for (int i = 0; i < R; ++i) {
                    s[i] = fmaf(__expf(dt * An[i]), s[i], dx * Bt[i]);
                    y = fmaf(s[i], Ct[i], y);
                }
            }
#pragma unroll
            for (int o = SC_NS / 2; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
            if (MODE == 1) dt_sum += dt;
            if (MODE != 1 && ns == 0) sy[t * SC_COLS + cl] = y + Dc * uv;
        }
        __syncthreads();
        for (int i = threadIdx.x; i < (MODE == 1 ? 0 : nt * SC_COLS); i += blockDim.x) {      // the chunk's outputs, gated
            const int t = i / SC_COLS, cc = i % SC_COLS;
            if (cc < ncol) {
                const float zz = st[t * PT + 2 * SC_COLS + cc];
                store_act(a.out, r0 + ch * SC_CH + t, c0 + cc, sy[i] * (zz / (1.f + expf(-zz))));
            }
        }
        __syncthreads();                                      // the stage is free for chunk ch + 2
    }
    float* Sout = MODE == 1 ? Sg : S;                         // MODE 0 and the last segment of MODE 2: the sequence's new state
    if (MODE == 2 && !last_seg) return;
#pragma unroll
    for (int i = 0; i < R; ++i) if (live && n0 + i < N) Sout[n0 + i] = s[i];
    if (MODE == 1 && ns == 0 && live) a.seg_dt[((size_t)e * SC_SEGS + seg) * a.inner + c] = dt_sum;
}
// Start state of every segment, in order: seg_state[k] holds S_local on entry and S_start(k) on exit (the last segment's end state is
// left by the scan proper).
__global__ void mamba1_seg_prefix_kernel(RaggedBatch rb, Mamba1Args a) {
    const int e = blockIdx.x, N = a.N, total = a.inner * N;
    const int len = rb.ent_len[e], slot = rb.ent_slot[e], nseg = (len + sc_seg_len(len) - 1) / sc_seg_len(len);
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < total; i += gridDim.y * blockDim.x) {
        const int c = i / N;
        float cur = a.state[(size_t)slot * total + i];
        const float An = a.A[i];
        for (int k = 0; k < nseg; ++k) {
            float* loc = a.seg_state + ((size_t)e * SC_SEGS + k) * total + i;
            const float l = *loc;
            *loc = cur;
            if (k + 1 < nseg) cur = fmaf(__expf(An * a.seg_dt[((size_t)e * SC_SEGS + k) * a.inner + c]), cur, l);
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------- mLSTM
// The gates first, block = (entry, head): per token the decay exp(fg + m_(t-1) - m_t), the input weight exp(ig - m_t) and exp(-m_t).
// The log gates of a chunk are computed side by side, the running maximum is a chain of additions and comparisons walked by one
// thread, the exponentials follow side by side.  Only this kernel reads and writes the carried maximum.
constexpr int MG_CH = 256;
__global__ void __launch_bounds__(MG_CH) mlstm_gates_kernel(RaggedBatch rb, MlstmArgs a, int T) {
    __shared__ float sig[MG_CH], sfg[MG_CH], sem[MG_CH + 1];
    __shared__ float m_run;
    const int e = blockIdx.x, h = blockIdx.y, H = a.H;
    const int len = rb.ent_len[e], r0 = rb.ent_row0[e], slot = rb.ent_slot[e];
    const int ic = a.col0 + 2 * H * a.d + 2 * H * a.dv + h, fc = ic + H;
    const float ib = a.i_b ? a.i_b[h] : 0.f, fb = a.f_b ? a.f_b[h] : 0.f;
    if (threadIdx.x == 0) m_run = a.m[(size_t)slot * H + h];
    for (int t0 = 0; t0 < len; t0 += MG_CH) {
        const int nt = min(MG_CH, len - t0), t = threadIdx.x;
        __syncthreads();
        if (t < nt) {
            const float* row = a.proj + (size_t)(r0 + t0 + t) * a.ld;
            sig[t] = a.gate_cap * tanhf((row[ic] + ib) / a.gate_cap);
            sfg[t] = log_sigmoid_f(a.gate_cap * tanhf((row[fc] + fb) / a.gate_cap));
        }
        __syncthreads();
        if (t == 0) {                       // the chain itself: one addition and one comparison per token
            float m = m_run;
            sem[MG_CH] = m;
#pragma unroll 8
            for (int k = 0; k < nt; ++k) {
                m = fmaxf(sfg[k] + m, sig[k]);
                sem[k] = m;
            }
            m_run = m;
        }
        __syncthreads();
        if (t < nt) {                       // what follows from it, side by side (the same roundings as a token-by-token walk: fg + m, then the difference)
            const float m_prev = t ? sem[t - 1] : sem[MG_CH], m_new = sem[t];
            float* g = a.gates + (size_t)(r0 + t0 + t) * H + h;
            g[0] = expf((sfg[t] + m_prev) - m_new); g[(size_t)T * H] = expf(sig[t] - m_new); g[(size_t)2 * T * H] = expf(-m_new);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) a.m[(size_t)slot * H + h] = m_run;
}

// The memory itself, block = (entry, head, SC_COLS columns); thread (pl, ns) owns rows n0 .. n0 + R - 1 of column p0 + pl in
// registers.  Columns 0 .. dv - 1 are those of S; column dv is the normaliser n (a value column whose value is always 1), kept in its
// own array.  Staged per chunk with cp.async, double-buffered: q, k (padded runs, see sc_idx), the block's value columns, decay and
// input weight per token.  The products S^T q and n . q of a chunk wait in shared memory and leave together; mlstm_out_kernel divides,
// normalises and gates.
template <int R, int MODE>
__global__ void __launch_bounds__(SC_COLS * SC_NS) mlstm_scan_kernel(RaggedBatch rb, MlstmArgs a, int T) {
    extern __shared__ __align__(16) float sm[];
    const int e = MODE == 0 ? blockIdx.x : blockIdx.x / SC_SEGS, seg = MODE == 0 ? 0 : blockIdx.x % SC_SEGS, h = blockIdx.y, p0 = blockIdx.z * SC_COLS;
    const int ns = threadIdx.x & (SC_NS - 1), pl = threadIdx.x / SC_NS, p = p0 + pl;
    const int H = a.H, d = a.d, dv = a.dv, DP = sc_pad(R), PT = 2 * DP + SC_COLS + 4;      // per staged token: q | k | v | decay, input weight
    const bool live = p <= dv, is_n = p == dv;
    const int full_len = rb.ent_len[e], slot = rb.ent_slot[e];
    const int seg_len = MODE == 0 ? full_len : sc_seg_len(full_len), seg0 = seg * seg_len;
    if (seg0 >= full_len) return;                             // (a short entry has fewer segments)
    const bool last_seg = seg0 + seg_len >= full_len;
    if (MODE == 1 && last_seg) return;                        // nothing follows the last segment: its end state is MODE 2's to leave
    const int len = min(seg_len, full_len - seg0), r0 = rb.ent_row0[e] + seg0;
    float* stage[2] = {sm, sm + SC_CH * PT};
    float* sy = sm + 2 * SC_CH * PT;                        // [CH][COLS]
    for (int i = threadIdx.x; i < 2 * SC_CH * PT; i += blockDim.x) sm[i] = 0.f;        // rows past d and columns past dv stay zero
    const int n0 = ns * R;
    float* col = is_n ? a.n + ((size_t)slot * H + h) * d : a.S + ((size_t)slot * H + h) * d * dv + (live ? p : 0);      // this thread's column, row stride cs
    const size_t cs = is_n ? 1 : (size_t)dv;
    // segments keep their states as [d, dv + 1] per head (the normaliser is column dv): MODE 1 leaves S_local there, MODE 2 starts from it
    float* gcol = MODE == 0 ? col : a.seg_state + (((size_t)e * SC_SEGS + seg) * H + h) * d * (dv + 1) + (live ? p : 0);
    const size_t gs = MODE == 0 ? cs : (size_t)(dv + 1);
    float s[R];
#pragma unroll
    for (int i = 0; i < R; ++i) s[i] = (live && n0 + i < d && MODE != 1) ? gcol[(size_t)(n0 + i) * gs] : 0.f;
    float dprod = 1.f;                                        // MODE 1: product of the segment's decays
    const int qc = a.col0 + h * d, kc = a.col0 + H * d + h * d, vc = a.col0 + 2 * H * d + h * dv;
    const int ncol = max(0, min(SC_COLS, dv - p0));          // value columns of S in this block
    __syncthreads();
    const bool wide = ((d | dv | a.ld | a.col0) & 3) == 0 && (R & 3) == 0 && ((size_t)a.proj & 15) == 0;
    auto fetch = [&](int ch, float* dst) {
        const int t0 = ch * SC_CH, nt = min(SC_CH, len - t0);
        if (wide) {
            const int nq = d >> 2, nv = ncol >> 2, per = 2 * nq + nv;
            for (int i = threadIdx.x; i < nt * per; i += blockDim.x) {
                const int t = i / per, k = i - t * per;
                const float* row = a.proj + (size_t)(r0 + t0 + t) * a.ld;
                float* d0 = dst + t * PT;
                if (k < nq) cp_async16s(d0 + sc_idx(4 * k, R), row + qc + 4 * k);
                else if (k < 2 * nq) cp_async16s(d0 + DP + sc_idx(4 * (k - nq), R), row + kc + 4 * (k - nq));
                else cp_async16s(d0 + 2 * DP + 4 * (k - 2 * nq), row + vc + p0 + 4 * (k - 2 * nq));
            }
        } else {
            const int per = 2 * d + ncol;
            for (int i = threadIdx.x; i < nt * per; i += blockDim.x) {
                const int t = i / per, k = i - t * per;
                const float* row = a.proj + (size_t)(r0 + t0 + t) * a.ld;
                float* d0 = dst + t * PT;
                if (k < d) cp_async4(d0 + sc_idx(k, R), row + qc + k);
                else if (k < 2 * d) cp_async4(d0 + DP + sc_idx(k - d, R), row + kc + k - d);
                else cp_async4(d0 + 2 * DP + k - 2 * d, row + vc + p0 + k - 2 * d);
            }
        }
        if (threadIdx.x < 2 * nt) {
            const int t = threadIdx.x >> 1, w = threadIdx.x & 1;
            cp_async4(dst + t * PT + 2 * DP + SC_COLS + w, a.gates + (size_t)w * T * H + (size_t)(r0 + t0 + t) * H + h);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const int nch = (len + SC_CH - 1) / SC_CH;
    fetch(0, stage[0]);
    for (int ch = 0; ch < nch; ++ch) {
        if (ch + 1 < nch) { fetch(ch + 1, stage[(ch + 1) & 1]); asm volatile("cp.async.wait_group 1;" ::: "memory"); }
        else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        const float* st = stage[ch & 1];
        const int nt = min(SC_CH, len - ch * SC_CH);
        const int tmax = (nt + 3) & ~3;                       // whole groups of four: a token past the end leaves the memory as it is
#pragma unroll 4
        for (int t = 0; t < tmax; ++t) {
            const float* tk = st + t * PT;
            const float dec = t < nt ? tk[2 * DP + SC_COLS] : 1.f, bv = t < nt ? tk[2 * DP + SC_COLS + 1] * (is_n ? 1.f : tk[2 * DP + pl]) : 0.f;
            const float* qt = tk + sc_idx(n0, R);
            const float* kt = qt + DP;
            float y0 = 0.f, y1 = 0.f;
            if constexpr ((R & 3) == 0) {
#pragma unroll
                for (int i = 0; i < R / 4; ++i) {
                    const float4 kk = reinterpret_cast<const float4*>(kt)[i], qq = reinterpret_cast<const float4*>(qt)[i];
                    s[4 * i] = fmaf(dec, s[4 * i], bv * kk.x); y0 = fmaf(s[4 * i], qq.x, y0);
                    s[4 * i + 1] = fmaf(dec, s[4 * i + 1], bv * kk.y); y1 = fmaf(s[4 * i + 1], qq.y, y1);
                    s[4 * i + 2] = fmaf(dec, s[4 * i + 2], bv * kk.z); y0 = fmaf(s[4 * i + 2], qq.z, y0);
                    s[4 * i + 3] = fmaf(dec, s[4 * i + 3], bv * kk.w); y1 = fmaf(s[4 * i + 3], qq.w, y1);
                }
            } else {
#pragma unroll
                for (int i = 0; i < R; ++i) {
                    s[i] = fmaf(dec, s[i], bv * kt[i]);
                    y0 = fmaf(s[i], qt[i], y0);
                }
            }
            if (MODE == 1) { dprod *= dec; continue; }
            float y = y0 + y1;
#pragma unroll
            for (int o = SC_NS / 2; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
            if (ns == 0) sy[t * SC_COLS + pl] = y * a.q_scale;
        }
        __syncthreads();
        for (int i = threadIdx.x; i < (MODE == 1 ? 0 : nt * SC_COLS); i += blockDim.x) {
            const int t = i / SC_COLS, pp = p0 + i % SC_COLS, r = r0 + ch * SC_CH + t;
            if (pp < dv) a.y[(size_t)r * H * dv + h * dv + pp] = sy[i];
            else if (pp == dv) a.gates[(size_t)3 * T * H + (size_t)r * H + h] = sy[i];
        }
        __syncthreads();                                      // the stage is free for chunk ch + 2
    }
    if (MODE == 2 && !last_seg) return;
    float* ocol = MODE == 1 ? gcol : col;                     // MODE 0 and the last segment of MODE 2: the sequence's new memory
    const size_t os = MODE == 1 ? gs : cs;
#pragma unroll
    for (int i = 0; i < R; ++i) if (live && n0 + i < d) ocol[(size_t)(n0 + i) * os] = s[i];
    if (MODE == 1 && threadIdx.x == 0 && blockIdx.z == 0) a.seg_decay[((size_t)e * SC_SEGS + seg) * H + h] = dprod;
}
// Start state of every segment, in order: seg_state[k] holds S_local on entry and S_start(k) on exit (the last segment's end state is
// left by the scan proper).
__global__ void mlstm_seg_prefix_kernel(RaggedBatch rb, MlstmArgs a) {
    const int e = blockIdx.x, h = blockIdx.y, d = a.d, dv = a.dv, np = d * (dv + 1);
    const int len = rb.ent_len[e], slot = rb.ent_slot[e], nseg = (len + sc_seg_len(len) - 1) / sc_seg_len(len);
    for (int i = blockIdx.z * blockDim.x + threadIdx.x; i < np; i += gridDim.z * blockDim.x) {
        const int row = i / (dv + 1), p = i % (dv + 1);
        float cur = p == dv ? a.n[((size_t)slot * a.H + h) * d + row] : a.S[(((size_t)slot * a.H + h) * d + row) * dv + p];
        for (int k = 0; k < nseg; ++k) {
            float* loc = a.seg_state + (((size_t)e * SC_SEGS + k) * a.H + h) * np + i;
            const float l = *loc;
            *loc = cur;
            if (k + 1 < nseg) cur = fmaf(a.seg_decay[((size_t)e * SC_SEGS + k) * a.H + h], cur, l);
        }
    }
}

// o = (S^T q) / (max(|n . q|, exp(-m)) + 1e-6);  out = o / sqrt(mean_dv(o^2) + eps) * norm_w * sigmoid(g): one warp per (row, head)
__global__ void mlstm_out_kernel(MlstmArgs a, int T) {
    const int lane = threadIdx.x & 31, wid = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (wid >= T * a.H) return;
    const int r = wid / a.H, h = wid % a.H, dv = a.dv;
    const float* y = a.y + (size_t)r * a.H * dv + h * dv;
    const float* g = a.proj + (size_t)r * a.ld + a.col0 + 2 * a.H * a.d + a.H * dv + h * dv;
    const float em = a.gates[(size_t)2 * T * a.H + (size_t)r * a.H + h], nq = a.gates[(size_t)3 * T * a.H + (size_t)r * a.H + h];
    const float den = 1.f / (fmaxf(fabsf(nq), em) + 1e-6f);
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) { const float o = y[c] * den; ss = fmaf(o, o, ss); }
    const float inv = 1.f / sqrtf(warp_sum(ss) / (float)dv + a.eps);
    for (int c = lane; c < dv; c += 32) store_act(a.out, r, h * dv + c, y[c] * den * inv * a.norm_w[h * dv + c] / (1.f + expf(-g[c])));
}

}  // namespace

int mamba1_scan_launch(cudaStream_t st, const RaggedBatch& rb, const Mamba1Args& a) {
    if (a.inner < 1 || a.N < 1 || a.N > SC_NS * 32 || a.dt_rank < 1 || !a.dt || !a.w_dtT) return -1000;
    static SmemOptIn seen_dt, seen_dt1;
    if (rb.T <= 8) {            // a decode step: one token per block row, so that every channel block of every token is a block of its own
        const size_t dsm = (size_t)a.dt_rank * sizeof(float);
        if (const int er = ensure_dyn_smem(mamba1_dt_kernel<1>, dsm, seen_dt1)) return er;
        mamba1_dt_kernel<1><<<dim3(rb.T, (a.inner + 127) / 128), 128, dsm, st>>>(a, rb.T);
    } else {
        const size_t dsm = (size_t)32 * a.dt_rank * sizeof(float);
        if (const int er = ensure_dyn_smem(mamba1_dt_kernel<32>, dsm, seen_dt)) return er;
        mamba1_dt_kernel<32><<<dim3((rb.T + 31) / 32, (a.inner + 127) / 128), 128, dsm, st>>>(a, rb.T);
    }
    if (const int er = last_err()) return er;
    const int nr = (a.N + SC_NS - 1) / SC_NS, R = nr <= 1 ? 1 : nr <= 2 ? 2 : nr <= 4 ? 4 : nr <= 8 ? 8 : nr <= 16 ? 16 : 32;
    const size_t smem = (size_t)(2 * SC_CH * (3 * SC_COLS + 2 * sc_pad(R)) + SC_CH * SC_COLS) * sizeof(float);
    const bool segs = a.seg_state != nullptr && a.max_len >= SC_SEG_MIN;
    const dim3 grid(segs ? rb.E * SC_SEGS : rb.E, (a.inner + SC_COLS - 1) / SC_COLS);
    auto run = [&](auto kern, SmemOptIn& seen) -> int {
        if (const int er = ensure_dyn_smem(kern, smem, seen)) return er;
        kern<<<grid, SC_COLS * SC_NS, smem, st>>>(rb, a);
        return last_err();
    };
    static SmemOptIn seen[3][6];
    auto scan = [&](auto mode) -> int {
        constexpr int M = decltype(mode)::value;
        switch (R) {
            case 1: return run(mamba1_scan_kernel<1, M>, seen[M][0]);
            case 2: return run(mamba1_scan_kernel<2, M>, seen[M][1]);
            case 4: return run(mamba1_scan_kernel<4, M>, seen[M][2]);
            case 8: return run(mamba1_scan_kernel<8, M>, seen[M][3]);
            case 16: return run(mamba1_scan_kernel<16, M>, seen[M][4]);
            default: return run(mamba1_scan_kernel<32, M>, seen[M][5]);
        }
    };
    if (!segs) return scan(std::integral_constant<int, 0>{});
    if (const int er = scan(std::integral_constant<int, 1>{})) return er;
    mamba1_seg_prefix_kernel<<<dim3(rb.E, std::max(1, std::min(128, (a.inner * a.N + 255) / 256))), 256, 0, st>>>(rb, a);
    if (const int er = last_err()) return er;
    return scan(std::integral_constant<int, 2>{});
}
int mamba1_launch_count(bool has_seg_scratch, int max_len) { return (has_seg_scratch && max_len >= SC_SEG_MIN) ? 4 : 2; }
size_t mamba1_seg_floats(int entries, int inner, int N) { return (size_t)entries * SC_SEGS * inner * ((size_t)N + 1); }
size_t mamba1_seg_dt_offset(int entries, int inner, int N) { return (size_t)entries * SC_SEGS * inner * (size_t)N; }

int mlstm_mixer_launch(cudaStream_t st, const RaggedBatch& rb, const MlstmArgs& a) {
    if (a.H < 1 || a.d < 1 || a.d > SC_NS * 32 || a.dv < 1 || !(a.gate_cap > 0.f) || !a.gates) return -1000;
    const int T = rb.T;
    mlstm_gates_kernel<<<dim3(rb.E, a.H), MG_CH, 0, st>>>(rb, a, T);
    int e = last_err();
    if (e) return e;
    const int nr = (a.d + SC_NS - 1) / SC_NS, R = nr <= 2 ? 2 : nr <= 4 ? 4 : nr <= 8 ? 8 : nr <= 16 ? 16 : 32;
    const size_t smem = (size_t)(2 * SC_CH * (2 * sc_pad(R) + SC_COLS + 4) + SC_CH * SC_COLS) * sizeof(float);
    const bool segs = a.seg_state != nullptr && a.max_len >= SC_SEG_MIN;
    const dim3 grid(segs ? rb.E * SC_SEGS : rb.E, a.H, (a.dv + 1 + SC_COLS - 1) / SC_COLS);
    auto run = [&](auto kern, SmemOptIn& seen) -> int {
        if (const int er = ensure_dyn_smem(kern, smem, seen)) return er;
        kern<<<grid, SC_COLS * SC_NS, smem, st>>>(rb, a, T);
        return last_err();
    };
    static SmemOptIn seen[3][5];
    auto scan = [&](auto mode) -> int {
        constexpr int M = decltype(mode)::value;
        switch (R) {
            case 2: return run(mlstm_scan_kernel<2, M>, seen[M][0]);
            case 4: return run(mlstm_scan_kernel<4, M>, seen[M][1]);
            case 8: return run(mlstm_scan_kernel<8, M>, seen[M][2]);
            case 16: return run(mlstm_scan_kernel<16, M>, seen[M][3]);
            default: return run(mlstm_scan_kernel<32, M>, seen[M][4]);
        }
    };
    if (!segs) e = scan(std::integral_constant<int, 0>{});
    else {
        if ((e = scan(std::integral_constant<int, 1>{}))) return e;
        mlstm_seg_prefix_kernel<<<dim3(rb.E, a.H, std::max(1, std::min(64, (a.d * (a.dv + 1) + 255) / 256))), 256, 0, st>>>(rb, a);
        if ((e = last_err())) return e;
        e = scan(std::integral_constant<int, 2>{});
    }
    if (e) return e;
    const int warps = T * a.H;
    mlstm_out_kernel<<<(warps + 3) / 4, 128, 0, st>>>(a, T);
    return last_err();
}
int mlstm_launch_count(bool has_seg_scratch, int max_len) { return (has_seg_scratch && max_len >= SC_SEG_MIN) ? 5 : 3; }
size_t mlstm_seg_floats(int entries, int H, int d, int dv) { return (size_t)entries * SC_SEGS * H * ((size_t)d * (dv + 1) + 1); }
size_t mlstm_seg_decay_offset(int entries, int H, int d, int dv) { return (size_t)entries * SC_SEGS * H * (size_t)d * (dv + 1); }

}  // namespace cb
