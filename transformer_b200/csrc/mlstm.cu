// A matrix memory with exponential gates (the mLSTM cell of xLSTM), token by token, state in float.
//
// Per head, with a state S [dim, vdim], n [dim] and a running maximum m (all zero when a sequence starts):
//
//   i_t = cap * tanh((zi_t + bi) / cap)                       log of the input gate
//   f_t = logsigmoid(cap * tanh((zf_t + bf) / cap))           log of the forget gate
//   m_t = max(f_t + m_{t-1}, i_t)
//   S_t = exp(f_t + m_{t-1} - m_t) S_{t-1} + exp(i_t - m_t) k_t v_t^T          n_t alike with k_t alone
//   o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)                      q scaled by dim^-1/2
//
// zi, zf are the gates' projections (float, computed by a product before this kernel), q, k, v the step's
// projections in the activation type.  Gates, decays, the state and the division are float on both paths.
//
// Work split: one block = one sequence x one head x 32 columns of v.  Lane = column, the block's 8 warps split
// the rows of S (warp w owns rows w, w + 8, ...: RPW registers per thread), so a block holds dim x 32 of the
// state in registers for all the tokens its sequence brings to the step, reads it once and writes it once.
// Every block keeps n and m for itself (they are cheap and every block needs them): the state holds one copy
// per block of columns, so that no block reads what another has already moved on.
//
// State of one (slot, head):  S [dim][vdim], then for each block of 32 columns: n [dim], m.
#include "common.cuh"

#define ML_WARPS 8
#define ML_COLS 32
#define ML_DENOM_FLOOR 1e-6f

struct MlstmArgs {
    const void* qkv;        // [nt, ld]: q heads | k heads | v heads (| anything else)
    const float* gates;     // [nt, 2 H]: zi of every head, then zf
    const float* bias;      // [2 H]
    float* state;           // [slots, H, state_size]
    float* out;             // [nt, H * vdim] unnormalized o
    const int* seq_start;   // [B + 1]
    const int* slots;       // [B]
    int ld, H, dim, vdim;
    float cap, qscale;
};

__device__ __forceinline__ float log_sigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

template <typename T, int RPW>
__global__ void __launch_bounds__(ML_WARPS * 32) mlstm_scan_kernel(const MlstmArgs a) {
    pdl_sync();
    constexpr int NQ = RPW * ML_WARPS / 32 > 0 ? RPW * ML_WARPS / 32 : 1;   // n entries per lane (dim <= 32 NQ)
    __shared__ float qk[2][2][RPW * ML_WARPS];      // [parity][q | k][dim]
    __shared__ float red[2][ML_WARPS][ML_COLS];
    const int b = blockIdx.x, h = blockIdx.y, cb = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, tid = threadIdx.x;
    const int dim = a.dim, vdim = a.vdim, H = a.H;
    const int col = cb * ML_COLS + lane;
    const bool has_col = col < vdim;
    const int t0 = a.seq_start[b], t1 = a.seq_start[b + 1];
    if (t0 >= t1) return;
    const int col_blocks = (vdim + ML_COLS - 1) / ML_COLS;
    const size_t state_size = (size_t)dim * vdim + (size_t)col_blocks * (dim + 1);
    float* S = a.state + ((size_t)a.slots[b] * H + h) * state_size;
    float* nvec = S + (size_t)dim * vdim + (size_t)cb * (dim + 1);
    float s[RPW], nq[NQ];
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
        const int r = warp + ML_WARPS * i;
        s[i] = (r < dim && has_col) ? S[(size_t)r * vdim + col] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < NQ; ++j) {
        const int r = lane + 32 * j;
        nq[j] = r < dim ? nvec[r] : 0.f;
    }
    float m = nvec[dim];
    const T* X = static_cast<const T*>(a.qkv);
    const float bi = a.bias[h], bf = a.bias[H + h], cap = a.cap, inv_cap = 1.0f / a.cap;
    // the next token's values are asked for while this one is computed
    auto fetch = [&](int t, float& q_, float& k_, float& v_, float& zi_, float& zf_) {
        const T* row = X + (size_t)t * a.ld;
        q_ = tid < dim ? ldf(row + (size_t)h * dim + tid) * a.qscale : 0.f;
        k_ = tid < dim ? ldf(row + (size_t)(H + h) * dim + tid) : 0.f;
        v_ = has_col ? ldf(row + (size_t)2 * H * dim + (size_t)h * vdim + col) : 0.f;
        zi_ = a.gates[(size_t)t * 2 * H + h];
        zf_ = a.gates[(size_t)t * 2 * H + H + h];
    };
    float q_r, k_r, v_r, zi, zf;
    fetch(t0, q_r, k_r, v_r, zi, zf);
    for (int t = t0; t < t1; ++t) {
        const int par = (t - t0) & 1;
        if (tid < RPW * ML_WARPS) {
            qk[par][0][tid] = q_r;
            qk[par][1][tid] = k_r;
        }
        const float v_c = v_r, zi_c = zi, zf_c = zf;
        if (t + 1 < t1) fetch(t + 1, q_r, k_r, v_r, zi, zf);
        __syncthreads();
        const float ig = cap * tanhf((zi_c + bi) * inv_cap);
        const float fg = log_sigmoid(cap * tanhf((zf_c + bf) * inv_cap));
        const float m_new = fmaxf(fg + m, ig);
        const float keep = expf(fg + m - m_new), take = expf(ig - m_new);
        m = m_new;
        const float tv = take * v_c;
        float part = 0.f;
#pragma unroll
        for (int i = 0; i < RPW; ++i) {
            const int r = warp + ML_WARPS * i;       // rows beyond dim hold zeros in qk and stay zero
            s[i] = keep * s[i] + qk[par][1][r] * tv;
            part += s[i] * qk[par][0][r];
        }
        red[par][warp][lane] = part;
        float dot = 0.f;
        if (warp == 0) {
#pragma unroll
            for (int j = 0; j < NQ; ++j) {
                const int r = lane + 32 * j;
                if (r < RPW * ML_WARPS) {
                    nq[j] = keep * nq[j] + take * qk[par][1][r];
                    dot += nq[j] * qk[par][0][r];
                }
            }
            dot = warp_sum(dot);
        }
        __syncthreads();
        if (warp == 0 && has_col) {
            float o = 0.f;
#pragma unroll
            for (int w = 0; w < ML_WARPS; ++w) o += red[par][w][lane];
            const float den = fmaxf(fabsf(dot), expf(-m)) + ML_DENOM_FLOOR;
            a.out[(size_t)t * H * vdim + (size_t)h * vdim + col] = o / den;
        }
    }
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
        const int r = warp + ML_WARPS * i;
        if (r < dim && has_col) S[(size_t)r * vdim + col] = s[i];
    }
    if (warp == 0) {
#pragma unroll
        for (int j = 0; j < NQ; ++j) {
            const int r = lane + 32 * j;
            if (r < dim) nvec[r] = nq[j];
        }
        if (lane == 0) nvec[dim] = m;
    }
}

// y[t, h, :] = o[t, h, :] / sqrt(mean_h(o^2) + eps) * w[h, :] * sigmoid(g[t, h, :])     one warp per (token, head)
template <typename T>
__global__ void __launch_bounds__(128)
mlstm_out_kernel(const float* __restrict__ o, const T* __restrict__ g, int ldg, const float* __restrict__ w,
                 T* __restrict__ y, int nt, int H, int vdim, float eps) {
    pdl_sync();
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (row >= nt * H) return;
    const int t = row / H, h = row - t * H;
    const float* orow = o + (size_t)t * H * vdim + (size_t)h * vdim;
    float ss = 0.f;
    for (int c = lane; c < vdim; c += 32) ss += orow[c] * orow[c];
    ss = warp_sum(ss);
    const float rs = 1.0f / sqrtf(ss / (float)vdim + eps);
    const T* grow = g + (size_t)t * ldg + (size_t)h * vdim;
    T* yrow = y + (size_t)t * H * vdim + (size_t)h * vdim;
    for (int c = lane; c < vdim; c += 32) {
        const float gate = 1.0f / (1.0f + expf(-ldf(grow + c)));
        stf(yrow + c, orow[c] * rs * w[(size_t)h * vdim + c] * gate);
    }
}

template <typename T>
static int mlstm_scan_launch(const MlstmArgs& a, int B, cudaStream_t s) {
    if (B < 0 || a.H <= 0 || a.dim <= 0 || a.vdim <= 0 || !(a.cap > 0.f)) return TB_ERR_ARG;
    if (a.dim > 32 * ML_WARPS) return TB_ERR_UNSUPPORTED;
    if (B == 0) return 0;
    dim3 grid(B, a.H, (a.vdim + ML_COLS - 1) / ML_COLS);
    const int rpw = (a.dim + ML_WARPS - 1) / ML_WARPS;
    if (rpw <= 4) TB_LAUNCH((mlstm_scan_kernel<T, 4>), grid, ML_WARPS * 32, 0, s, a);
    else if (rpw <= 8) TB_LAUNCH((mlstm_scan_kernel<T, 8>), grid, ML_WARPS * 32, 0, s, a);
    else if (rpw <= 16) TB_LAUNCH((mlstm_scan_kernel<T, 16>), grid, ML_WARPS * 32, 0, s, a);
    else TB_LAUNCH((mlstm_scan_kernel<T, 32>), grid, ML_WARPS * 32, 0, s, a);
    return tb_last_error();
}

extern "C" {
// Floats of state per (slot, head) for the given sizes.
int tb_mlstm_state_size(int dim, int vdim) {
    return dim * vdim + (vdim + ML_COLS - 1) / ML_COLS * (dim + 1);
}
#define TB_MLSTM(SFX, T)                                                                                              \
    int tb_mlstm_scan_##SFX(const void* qkv, const float* gates, const float* bias, float* state, float* out,         \
                            const int* seq_start, const int* slots, int B, int ld, int H, int dim, int vdim, float cap, \
                            float qscale, cudaStream_t s) {                                                           \
        MlstmArgs a{qkv, gates, bias, state, out, seq_start, slots, ld, H, dim, vdim, cap, qscale};                   \
        return mlstm_scan_launch<T>(a, B, s);                                                                         \
    }                                                                                                                 \
    int tb_mlstm_out_##SFX(const float* o, const void* g, int ldg, const float* w, void* y, int nt, int H, int vdim,  \
                           float eps, cudaStream_t s) {                                                               \
        if (nt < 0 || H <= 0 || vdim <= 0) return TB_ERR_ARG;                                                         \
        if (nt == 0) return 0;                                                                                        \
        TB_LAUNCH((mlstm_out_kernel<T>), (nt * H + 3) / 4, 128, 0, s, o, (const T*)g, ldg, w, (T*)y, nt, H, vdim, eps); \
        return tb_last_error();                                                                                       \
    }
TB_MLSTM(f32, float)
TB_MLSTM(bf16, __nv_bfloat16)
}

#include "tape.h"
TB_TAPE_REGISTER(tb_mlstm_scan_f32)
TB_TAPE_REGISTER(tb_mlstm_scan_bf16)
TB_TAPE_REGISTER(tb_mlstm_out_f32)
TB_TAPE_REGISTER(tb_mlstm_out_bf16)
