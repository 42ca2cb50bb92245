// Recurrent mixers of ragged-batch steps whose state is carried per sequence slot in f32 (see ragged.cuh):
//   * the selective scan with a state per channel (Mamba-1): decay exp(dt_c A[c, n]) per channel and state entry;
//   * the matrix memory with exponential gates and a running maximum (mLSTM): a scalar decay per head and token.
// Both walk a portion token by token; a thread keeps its share of the state in registers for the whole portion, the step inputs of
// SC_CH tokens at a time are staged in shared memory, and everything that enters the recurrence (step sizes, softplus, decays,
// gates, the running maximum) is computed in f32 when the chunk lands.  A row's result depends on its own sequence only: the
// split of the state over lanes and the order of the lane sums are launch constants.
#include "ragged.cuh"
#include "ragged_dev.cuh"

#include <algorithm>

namespace cb {

namespace {

constexpr int SC_NS = 8;        // lanes that share one channel (Mamba-1) / one value column (mLSTM): each owns a contiguous slice of the state
constexpr int SC_COLS = 16;     // channels / value columns per block -> 128 threads
constexpr int SC_CH = 16;       // tokens staged per chunk

inline int last_err() { return (int)cudaGetLastError(); }

__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float log_sigmoid_f(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

// ---------------------------------------------------------------------------------------------------------------- Mamba-1
// Block = (entry, SC_COLS channels); thread (cl, ns) owns the state entries n = ns * R .. ns * R + R - 1 of channel c0 + cl.
// Staged per chunk: u [CH][COLS], dt [CH][COLS] (softplus of the low-rank projection, computed here), B and C [CH][NP].
template <int R>
__global__ void __launch_bounds__(SC_COLS * SC_NS) mamba1_scan_kernel(RaggedBatch rb, Mamba1Args a) {
    extern __shared__ __align__(16) float sm[];
    const int e = blockIdx.x, c0 = blockIdx.y * SC_COLS;
    const int ns = threadIdx.x & (SC_NS - 1), cl = threadIdx.x / SC_NS, c = c0 + cl;
    const int N = a.N, NP = SC_NS * R, Rk = a.dt_rank;
    const bool live = c < a.inner;
    const int len = rb.ent_len[e], r0 = rb.ent_row0[e], slot = rb.ent_slot[e];
    float* su = sm;                         // [CH][COLS]
    float* sdt = su + SC_CH * SC_COLS;      // [CH][COLS]
    float* sB = sdt + SC_CH * SC_COLS;      // [CH][NP]
    float* sC = sB + SC_CH * NP;            // [CH][NP]
    float* slow = sC + SC_CH * NP;          // [CH][Rk]
    float* swdt = slow + SC_CH * Rk;        // [COLS][Rk]
    const int n0 = ns * R;
    float s[R], An[R];
    float* S = a.state + ((size_t)slot * a.inner + (live ? c : 0)) * N;
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const bool ok = live && n0 + i < N;
        s[i] = ok ? S[n0 + i] : 0.f;
        An[i] = ok ? a.A[(size_t)c * N + n0 + i] : 0.f;
    }
    for (int i = threadIdx.x; i < SC_COLS * Rk; i += blockDim.x) {
        const int cc = c0 + i / Rk;
        swdt[i] = cc < a.inner ? a.w_dt[(size_t)cc * Rk + i % Rk] : 0.f;
    }
    const float Dc = live ? a.D[c] : 0.f;
    for (int t0 = 0; t0 < len; t0 += SC_CH) {
        const int nt = min(SC_CH, len - t0);
        __syncthreads();                    // the last chunk's readers are done
        for (int i = threadIdx.x; i < nt * SC_COLS; i += blockDim.x) {
            const int t = i / SC_COLS, cc = c0 + i % SC_COLS;
            su[i] = cc < a.inner ? a.u[(size_t)(r0 + t0 + t) * a.ldu + cc] : 0.f;
        }
        for (int i = threadIdx.x; i < nt * NP; i += blockDim.x) {
            const int t = i / NP, n = i % NP;
            const float* lr = a.low + (size_t)(r0 + t0 + t) * a.ldl + Rk;
            sB[i] = n < N ? lr[n] : 0.f;
            sC[i] = n < N ? lr[N + n] : 0.f;
        }
        for (int i = threadIdx.x; i < nt * Rk; i += blockDim.x) slow[i] = a.low[(size_t)(r0 + t0 + i / Rk) * a.ldl + i % Rk];
        __syncthreads();
        for (int i = threadIdx.x; i < nt * SC_COLS; i += blockDim.x) {       // step sizes: a dt_rank-long dot per (token, channel), in order
            const int t = i / SC_COLS, cc = i % SC_COLS;
            float z = 0.f;
            for (int k = 0; k < Rk; ++k) z = fmaf(swdt[cc * Rk + k], slow[t * Rk + k], z);
            sdt[i] = c0 + cc < a.inner ? softplus_f(z + a.dt_b[c0 + cc]) : 0.f;
        }
        __syncthreads();
        for (int t = 0; t < nt; ++t) {
            const float dt = sdt[t * SC_COLS + cl], uv = su[t * SC_COLS + cl], dx = dt * uv;
            const float* Bt = sB + t * NP + n0;
            const float* Ct = sC + t * NP + n0;
            float y = 0.f;
#pragma unroll
            for (int i = 0; i < R; ++i) {
                s[i] = fmaf(__expf(dt * An[i]), s[i], dx * Bt[i]);
                y = fmaf(s[i], Ct[i], y);
            }
#pragma unroll
            for (int o = SC_NS / 2; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
            if (ns == 0 && live) {
                const int r = r0 + t0 + t;
                const float zz = a.z[(size_t)r * a.ldz + c];
                store_act(a.out, r, c, (y + Dc * uv) * (zz / (1.f + expf(-zz))));
            }
        }
    }
#pragma unroll
    for (int i = 0; i < R; ++i) if (live && n0 + i < N) S[n0 + i] = s[i];
}

// ---------------------------------------------------------------------------------------------------------------- mLSTM
// The gates first, block = (entry, head): per token the decay exp(fg + m_(t-1) - m_t), the input weight exp(ig - m_t) and exp(-m_t).
// The log gates of a chunk are computed side by side, the running maximum is a chain of additions and comparisons walked by one
// thread, the exponentials follow side by side.  Only this kernel reads and writes the carried maximum.
constexpr int MG_CH = 256;
__global__ void __launch_bounds__(MG_CH) mlstm_gates_kernel(RaggedBatch rb, MlstmArgs a, int T) {
    __shared__ float sig[MG_CH], sfg[MG_CH], sa[MG_CH], sb[MG_CH], sem[MG_CH];
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
        if (t == 0) {
            float m = m_run;
            for (int k = 0; k < nt; ++k) {
                const float mn = fmaxf(sfg[k] + m, sig[k]);
                sa[k] = sfg[k] + m - mn; sb[k] = sig[k] - mn; sem[k] = -mn;
                m = mn;
            }
            m_run = m;
        }
        __syncthreads();
        if (t < nt) {
            float* g = a.gates + (size_t)(r0 + t0 + t) * H + h;
            g[0] = expf(sa[t]); g[(size_t)T * H] = expf(sb[t]); g[(size_t)2 * T * H] = expf(sem[t]);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) a.m[(size_t)slot * H + h] = m_run;
}

// The memory itself, block = (entry, head, SC_COLS columns); thread (pl, ns) owns rows n0 .. n0 + R - 1 of column p0 + pl.  Columns
// 0 .. dv - 1 are those of S; column dv is the normaliser n (a value column whose value is always 1), kept in its own array.
// Staged per chunk: q (scaled), k [CH][DP], v [CH][COLS], decay and input weight per token.  The products S^T q and n . q go to
// scratch; mlstm_out_kernel divides, normalises and gates.
template <int R>
__global__ void __launch_bounds__(SC_COLS * SC_NS) mlstm_scan_kernel(RaggedBatch rb, MlstmArgs a, int T) {
    extern __shared__ __align__(16) float sm[];
    __shared__ float sa[SC_CH], sb[SC_CH];
    const int e = blockIdx.x, h = blockIdx.y, p0 = blockIdx.z * SC_COLS;
    const int ns = threadIdx.x & (SC_NS - 1), pl = threadIdx.x / SC_NS, p = p0 + pl;
    const int H = a.H, d = a.d, dv = a.dv, DP = SC_NS * R;
    const bool live = p <= dv, is_n = p == dv;
    const int len = rb.ent_len[e], r0 = rb.ent_row0[e], slot = rb.ent_slot[e];
    float* sq = sm;                         // [CH][DP]
    float* sk = sq + SC_CH * DP;            // [CH][DP]
    float* sv = sk + SC_CH * DP;            // [CH][COLS]
    const int n0 = ns * R;
    float* col = is_n ? a.n + ((size_t)slot * H + h) * d : a.S + ((size_t)slot * H + h) * d * dv + p;      // this thread's column, row stride cs
    const size_t cs = is_n ? 1 : (size_t)dv;
    float s[R];
#pragma unroll
    for (int i = 0; i < R; ++i) s[i] = (live && n0 + i < d) ? col[(size_t)(n0 + i) * cs] : 0.f;
    const int qc = a.col0 + h * d, kc = a.col0 + H * d + h * d, vc = a.col0 + 2 * H * d + h * dv;
    for (int t0 = 0; t0 < len; t0 += SC_CH) {
        const int nt = min(SC_CH, len - t0);
        __syncthreads();
        for (int i = threadIdx.x; i < nt * DP; i += blockDim.x) {
            const int t = i / DP, n = i % DP;
            const float* row = a.proj + (size_t)(r0 + t0 + t) * a.ld;
            sq[i] = n < d ? row[qc + n] * a.q_scale : 0.f;
            sk[i] = n < d ? row[kc + n] : 0.f;
        }
        for (int i = threadIdx.x; i < nt * SC_COLS; i += blockDim.x) {
            const int t = i / SC_COLS, pp = p0 + i % SC_COLS;
            sv[i] = pp < dv ? a.proj[(size_t)(r0 + t0 + t) * a.ld + vc + pp] : pp == dv ? 1.f : 0.f;
        }
        if (threadIdx.x < nt) {
            const float* g = a.gates + (size_t)(r0 + t0 + threadIdx.x) * H + h;
            sa[threadIdx.x] = g[0]; sb[threadIdx.x] = g[(size_t)T * H];
        }
        __syncthreads();
        for (int t = 0; t < nt; ++t) {
            const float dec = sa[t], bv = sb[t] * sv[t * SC_COLS + pl];
            const float* kt = sk + t * DP + n0;
            const float* qt = sq + t * DP + n0;
            float y = 0.f;
#pragma unroll
            for (int i = 0; i < R; ++i) {
                s[i] = fmaf(dec, s[i], bv * kt[i]);
                y = fmaf(s[i], qt[i], y);
            }
#pragma unroll
            for (int o = SC_NS / 2; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
            if (ns == 0 && live) {
                if (is_n) a.gates[(size_t)3 * T * H + (size_t)(r0 + t0 + t) * H + h] = y;
                else a.y[(size_t)(r0 + t0 + t) * H * dv + h * dv + p] = y;
            }
        }
    }
#pragma unroll
    for (int i = 0; i < R; ++i) if (live && n0 + i < d) col[(size_t)(n0 + i) * cs] = s[i];
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
    if (a.inner < 1 || a.N < 1 || a.N > SC_NS * 32 || a.dt_rank < 1) return -1000;
    const int nr = (a.N + SC_NS - 1) / SC_NS, R = nr <= 1 ? 1 : nr <= 2 ? 2 : nr <= 4 ? 4 : nr <= 8 ? 8 : nr <= 16 ? 16 : 32;
    const size_t smem = (size_t)(2 * SC_CH * SC_COLS + 2 * SC_CH * SC_NS * R + SC_CH * a.dt_rank + SC_COLS * a.dt_rank) * sizeof(float);
    if (smem > 200 * 1024) return -1000;
    const dim3 grid(rb.E, (a.inner + SC_COLS - 1) / SC_COLS);
    auto run = [&](auto kern, SmemOptIn& seen) -> int {
        if (const int er = ensure_dyn_smem(kern, smem, seen)) return er;
        kern<<<grid, SC_COLS * SC_NS, smem, st>>>(rb, a);
        return last_err();
    };
    static SmemOptIn seen[6];
    switch (R) {
        case 1: return run(mamba1_scan_kernel<1>, seen[0]);
        case 2: return run(mamba1_scan_kernel<2>, seen[1]);
        case 4: return run(mamba1_scan_kernel<4>, seen[2]);
        case 8: return run(mamba1_scan_kernel<8>, seen[3]);
        case 16: return run(mamba1_scan_kernel<16>, seen[4]);
        default: return run(mamba1_scan_kernel<32>, seen[5]);
    }
}

int mlstm_mixer_launch(cudaStream_t st, const RaggedBatch& rb, const MlstmArgs& a) {
    if (a.H < 1 || a.d < 1 || a.d > SC_NS * 32 || a.dv < 1 || !(a.gate_cap > 0.f) || !a.gates) return -1000;
    const int T = rb.T;
    mlstm_gates_kernel<<<dim3(rb.E, a.H), MG_CH, 0, st>>>(rb, a, T);
    int e = last_err();
    if (e) return e;
    const int nr = (a.d + SC_NS - 1) / SC_NS, R = nr <= 2 ? 2 : nr <= 4 ? 4 : nr <= 8 ? 8 : nr <= 16 ? 16 : 32;
    const size_t smem = (size_t)(2 * SC_CH * SC_NS * R + SC_CH * SC_COLS) * sizeof(float);
    const dim3 grid(rb.E, a.H, (a.dv + 1 + SC_COLS - 1) / SC_COLS);
    auto run = [&](auto kern, SmemOptIn& seen) -> int {
        if (const int er = ensure_dyn_smem(kern, smem, seen)) return er;
        kern<<<grid, SC_COLS * SC_NS, smem, st>>>(rb, a, T);
        return last_err();
    };
    static SmemOptIn seen[5];
    switch (R) {
        case 2: e = run(mlstm_scan_kernel<2>, seen[0]); break;
        case 4: e = run(mlstm_scan_kernel<4>, seen[1]); break;
        case 8: e = run(mlstm_scan_kernel<8>, seen[2]); break;
        case 16: e = run(mlstm_scan_kernel<16>, seen[3]); break;
        default: e = run(mlstm_scan_kernel<32>, seen[4]); break;
    }
    if (e) return e;
    const int warps = T * a.H;
    mlstm_out_kernel<<<(warps + 3) / 4, 128, 0, st>>>(a, T);
    return last_err();
}

}  // namespace cb
