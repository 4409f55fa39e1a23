// A gated delta rule with one decay per key channel, token by token, state in float.
//
// Per head h (its queries and keys come from key head h / (H / G)), with a state S [dim, vdim] that is zero when a
// sequence starts:
//
//   S <- diag(g_t) S;    u = beta_t (v_t - S^T k_t);    S <- S + k_t u^T;    o_t = S^T q_t
//
// What enters the recurrence is made by the kernel before it (delta_prep_kernel), in float on both paths:
//   q, k, v = silu(causal convolution over time of the step's projections, per channel, `taps` wide);
//   q and k unit vectors per head (x / sqrt(sum x^2 + 1e-6)), q also times dim^-1/2;
//   g = exp(-exp(A_log[h]) * softplus(a + dt_bias))  per head and key channel;   beta = sigmoid(b)  per head.
// The last taps - 1 inputs of every channel are state as well, so that a sequence may arrive in pieces.
//
// State of one slot (floats): S [H][dim][vdim], then the convolution's inputs [taps - 1][C], C = 2 G dim + H vdim.
//
// The scan reads o_t = (gS)^T q + u (k . q) from the SAME pass over the state that gives (gS)^T k, so a token costs
// one pass for the two sums, a reduction over the four lanes that share a column, and one pass for the update.
// Work split of the scan: a block = one sequence x one head x 32 columns of the state; a column belongs to four
// adjacent lanes, which split the rows (chunks of four rows, interleaved), RPT rows each in registers.
#include "common.cuh"

#define CD_UNIT_EPS 1e-6f
#define CD_SPLIT 4
#define CD_COLS 32
#define CD_THREADS (CD_SPLIT * CD_COLS)
#define CD_MAX_TAPS 16

struct DeltaPrepArgs {
    const void* z;          // [nt, ldz]: q (G dim) | k (G dim) | v (H vdim) | whatever else the product made
    const float* wconv;     // [C, taps], the last column is the current token's
    float* state;           // [slots, state_stride]
    const float* a;         // [nt, H dim]  pre-activation of the decay
    const float* dt_bias;   // [H dim]
    const float* A_log;     // [H]
    const float* bz;        // [nt, H]      pre-activation of beta
    float* qkv;             // out [nt, C]
    float* decay;           // out [nt, H dim]
    float* beta;            // out [nt, H]
    float* kq;              // out [nt, H]  k . q of the head's key head (after the unit norms and the scale)
    const int* tok_seq;
    const int* seq_start;
    const int* slots;
    long long state_stride, conv_offset;
    int ldz, G, H, dim, vdim, taps, update_state;
};

__device__ __forceinline__ float cd_softplus(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }

template <typename T>
__global__ void __launch_bounds__(256) delta_prep_kernel(const DeltaPrepArgs p) {
    pdl_sync();
    extern __shared__ float y[];        // [C] the convolution's outputs after silu
    const int t = blockIdx.x;
    const int b = p.tok_seq[t];
    const int li = t - p.seq_start[b];                  // index of the token among its sequence's tokens of the step
    const int C = 2 * p.G * p.dim + p.H * p.vdim, taps = p.taps;
    const T* z = static_cast<const T*>(p.z);
    float* cs = p.state + (size_t)p.slots[b] * p.state_stride + p.conv_offset;     // [taps - 1][C]
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float acc = 0.f, old[CD_MAX_TAPS];
        for (int j = 0; j < taps; ++j) {
            const int back = taps - 1 - j, s = li - back;
            const float x = s >= 0 ? ldf(z + (size_t)(t - back) * p.ldz + c) : cs[(size_t)(taps - 1 + s) * C + c];
            old[j] = x;
            acc += p.wconv[(size_t)c * taps + j] * x;
        }
        y[c] = acc / (1.0f + expf(-acc));
        if (p.update_state)         // a step of one token per sequence: this thread alone touches its channel's state
            for (int r = 0; r + 1 < taps; ++r) cs[(size_t)r * C + c] = old[r + 1];
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int dim = p.dim, gd = p.G * p.dim;
    float* out = p.qkv + (size_t)t * C;
    for (int g = warp; g < p.G; g += nw) {
        const float* q = y + g * dim;
        const float* k = y + gd + g * dim;
        float sq = 0.f, sk = 0.f, dot = 0.f;
        for (int c = lane; c < dim; c += 32) {
            sq += q[c] * q[c];
            sk += k[c] * k[c];
            dot += q[c] * k[c];
        }
        sq = warp_sum(sq);
        sk = warp_sum(sk);
        dot = warp_sum(dot);
        const float iq = rsqrtf((float)dim) / sqrtf(sq + CD_UNIT_EPS), ik = 1.0f / sqrtf(sk + CD_UNIT_EPS);
        for (int c = lane; c < dim; c += 32) {
            out[g * dim + c] = q[c] * iq;
            out[gd + g * dim + c] = k[c] * ik;
        }
        const int per = p.H / p.G;
        if (lane < per) p.kq[(size_t)t * p.H + g * per + lane] = dot * iq * ik;
        for (int h = lane + 32; h < per; h += 32) p.kq[(size_t)t * p.H + g * per + h] = dot * iq * ik;
    }
    for (int c = 2 * gd + threadIdx.x; c < C; c += blockDim.x) out[c] = y[c];
    for (int i = threadIdx.x; i < p.H * dim; i += blockDim.x) {
        const int h = i / dim;
        p.decay[(size_t)t * p.H * dim + i] =
            expf(-expf(p.A_log[h]) * cd_softplus(p.a[(size_t)t * p.H * dim + i] + p.dt_bias[i]));
    }
    if (threadIdx.x < p.H) p.beta[(size_t)t * p.H + threadIdx.x] = 1.0f / (1.0f + expf(-p.bz[(size_t)t * p.H + threadIdx.x]));
    for (int h = threadIdx.x + blockDim.x; h < p.H; h += blockDim.x)
        p.beta[(size_t)t * p.H + h] = 1.0f / (1.0f + expf(-p.bz[(size_t)t * p.H + h]));
}

// After a step that brought a sequence more than one token: the last taps - 1 inputs of every channel, from the
// step's rows and, where the step was shorter than that, from what the state held.
template <typename T>
__global__ void __launch_bounds__(256) delta_conv_state_kernel(const DeltaPrepArgs p) {
    pdl_sync();
    const int b = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    const int C = 2 * p.G * p.dim + p.H * p.vdim, keep = p.taps - 1;
    if (c >= C) return;
    const int t0 = p.seq_start[b], n = p.seq_start[b + 1] - t0;
    if (n <= 0) return;
    const T* z = static_cast<const T*>(p.z);
    float* cs = p.state + (size_t)p.slots[b] * p.state_stride + p.conv_offset;
    float fresh[CD_MAX_TAPS];
    for (int r = 0; r < keep; ++r) {
        const int li = n - keep + r;
        fresh[r] = li >= 0 ? ldf(z + (size_t)(t0 + li) * p.ldz + c) : cs[(size_t)(keep + li) * C + c];
    }
    for (int r = 0; r < keep; ++r) cs[(size_t)r * C + c] = fresh[r];
}

struct DeltaScanArgs {
    const float* qkv;       // [nt, C]
    const float* decay;     // [nt, H dim]
    const float* beta;      // [nt, H]
    const float* kq;        // [nt, H]
    float* state;           // [slots, state_stride], S first
    float* out;             // [nt, H vdim]
    const int* seq_start;
    const int* slots;
    long long state_stride;
    int G, H, dim, vdim;
};

template <int RPT>
__global__ void __launch_bounds__(CD_THREADS) delta_scan_kernel(const DeltaScanArgs a) {
    pdl_sync();
    constexpr int DP = RPT * CD_SPLIT;                  // rows the block's lanes cover (dim rounded up)
    constexpr int NF = (3 * DP + CD_THREADS - 1) / CD_THREADS;
    __shared__ __align__(16) float sm[2][3][DP];        // [parity][q | k | g][row]
    const int b = blockIdx.x, h = blockIdx.y;
    const int tid = threadIdx.x, part = tid & (CD_SPLIT - 1);
    const int col = blockIdx.z * CD_COLS + (tid >> 2);
    const int dim = a.dim, vdim = a.vdim, H = a.H;
    const bool has_col = col < vdim;
    const int t0 = a.seq_start[b], t1 = a.seq_start[b + 1];
    if (t0 >= t1) return;
    const int g = h / (H / a.G), gd = a.G * dim, C = 2 * gd + H * vdim;
    float* S = a.state + (size_t)a.slots[b] * a.state_stride + (size_t)h * dim * vdim;
    float s[RPT];
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
        const int r = ((i >> 2) * CD_SPLIT + part) * 4 + (i & 3);
        s[i] = (r < dim && has_col) ? S[(size_t)r * vdim + col] : 0.f;
    }
    // the next token's vectors are asked for while this one is computed
    float f[NF], v_r, beta_r, kq_r;
    auto fetch = [&](int t) {
#pragma unroll
        for (int j = 0; j < NF; ++j) {
            const int idx = tid + j * CD_THREADS, which = idx / DP, r = idx - which * DP;
            float x = which == 2 ? 1.f : 0.f;
            if (which < 3 && r < dim)
                x = which == 0 ? a.qkv[(size_t)t * C + g * dim + r]
                  : which == 1 ? a.qkv[(size_t)t * C + gd + g * dim + r]
                               : a.decay[((size_t)t * H + h) * dim + r];
            f[j] = x;
        }
        v_r = has_col ? a.qkv[(size_t)t * C + 2 * gd + (size_t)h * vdim + col] : 0.f;
        beta_r = a.beta[(size_t)t * H + h];
        kq_r = a.kq[(size_t)t * H + h];
    };
    fetch(t0);
    for (int t = t0; t < t1; ++t) {
        const int par = (t - t0) & 1;
        float* stage = &sm[par][0][0];
#pragma unroll
        for (int j = 0; j < NF; ++j) {
            const int idx = tid + j * CD_THREADS;
            if (idx < 3 * DP) stage[idx] = f[j];
        }
        const float v_c = v_r, beta_c = beta_r, kq_c = kq_r;
        if (t + 1 < t1) fetch(t + 1);
        __syncthreads();
        const float4* Q4 = reinterpret_cast<const float4*>(&sm[par][0][0]);
        const float4* K4 = reinterpret_cast<const float4*>(&sm[par][1][0]);
        const float4* G4 = reinterpret_cast<const float4*>(&sm[par][2][0]);
        float dk = 0.f, dq = 0.f;
#pragma unroll
        for (int i4 = 0; i4 < RPT / 4; ++i4) {
            const int ch = i4 * CD_SPLIT + part;
            const float4 q = Q4[ch], k = K4[ch], gg = G4[ch];
            float* si = s + i4 * 4;
            si[0] *= gg.x; si[1] *= gg.y; si[2] *= gg.z; si[3] *= gg.w;
            dk += si[0] * k.x + si[1] * k.y + si[2] * k.z + si[3] * k.w;
            dq += si[0] * q.x + si[1] * q.y + si[2] * q.z + si[3] * q.w;
        }
        dk += __shfl_xor_sync(0xffffffffu, dk, 1);
        dq += __shfl_xor_sync(0xffffffffu, dq, 1);
        dk += __shfl_xor_sync(0xffffffffu, dk, 2);
        dq += __shfl_xor_sync(0xffffffffu, dq, 2);
        const float u = beta_c * (v_c - dk);
#pragma unroll
        for (int i4 = 0; i4 < RPT / 4; ++i4) {
            const float4 k = K4[i4 * CD_SPLIT + part];
            float* si = s + i4 * 4;
            si[0] += k.x * u; si[1] += k.y * u; si[2] += k.z * u; si[3] += k.w * u;
        }
        if (part == 0 && has_col) a.out[((size_t)t * H + h) * vdim + col] = dq + u * kq_c;
    }
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
        const int r = ((i >> 2) * CD_SPLIT + part) * 4 + (i & 3);
        if (r < dim && has_col) S[(size_t)r * vdim + col] = s[i];
    }
}

template <typename T>
static int delta_prep_launch(const DeltaPrepArgs& p, int nt, int B, cudaStream_t s) {
    if (nt < 0 || B < 0 || p.G <= 0 || p.H <= 0 || p.H % p.G || p.dim <= 0 || p.vdim <= 0) return TB_ERR_ARG;
    if (p.taps < 1 || p.taps > CD_MAX_TAPS) return TB_ERR_UNSUPPORTED;
    const int C = 2 * p.G * p.dim + p.H * p.vdim;
    const size_t smem = (size_t)C * sizeof(float);
    if (smem > 200 * 1024) return TB_ERR_UNSUPPORTED;
    if (nt == 0) return 0;
    static size_t configured = 0;
    if (smem > 48 * 1024 && smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(delta_prep_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    TB_LAUNCH((delta_prep_kernel<T>), nt, 256, smem, s, p);
    int rc = tb_last_error();
    if (rc || p.update_state || p.taps == 1) return rc;
    dim3 grid(B, (C + 255) / 256);
    TB_LAUNCH((delta_conv_state_kernel<T>), grid, 256, 0, s, p);
    return tb_last_error();
}

static int delta_scan_launch(const DeltaScanArgs& a, int B, cudaStream_t s) {
    if (B < 0 || a.G <= 0 || a.H <= 0 || a.H % a.G || a.dim <= 0 || a.vdim <= 0) return TB_ERR_ARG;
    if (a.dim > 256) return TB_ERR_UNSUPPORTED;
    if (B == 0) return 0;
    dim3 grid(B, a.H, (a.vdim + CD_COLS - 1) / CD_COLS);
    const int rpt = (a.dim + CD_SPLIT - 1) / CD_SPLIT;
    if (rpt <= 4) TB_LAUNCH((delta_scan_kernel<4>), grid, CD_THREADS, 0, s, a);
    else if (rpt <= 8) TB_LAUNCH((delta_scan_kernel<8>), grid, CD_THREADS, 0, s, a);
    else if (rpt <= 16) TB_LAUNCH((delta_scan_kernel<16>), grid, CD_THREADS, 0, s, a);
    else if (rpt <= 32) TB_LAUNCH((delta_scan_kernel<32>), grid, CD_THREADS, 0, s, a);
    else TB_LAUNCH((delta_scan_kernel<64>), grid, CD_THREADS, 0, s, a);
    return tb_last_error();
}

extern "C" {
// Floats of state per slot: the matrix memory of every head, then the convolution's last inputs.
int tb_delta_state_size(int G, int H, int dim, int vdim, int taps) {
    return H * dim * vdim + (taps - 1) * (2 * G * dim + H * vdim);
}
#define TB_DELTA_PREP(SFX, T)                                                                                         \
    int tb_delta_prep_##SFX(const void* z, int ldz, const float* wconv, float* state, const float* a,                 \
                            const float* dt_bias, const float* A_log, const float* bz, float* qkv, float* decay,      \
                            float* beta, float* kq, const int* tok_seq, const int* seq_start, const int* slots,       \
                            int nt, int B, int G, int H, int dim, int vdim, int taps, int update_state,               \
                            cudaStream_t s) {                                                                         \
        DeltaPrepArgs p{z, wconv, state, a, dt_bias, A_log, bz, qkv, decay, beta, kq, tok_seq, seq_start, slots,      \
                        (long long)tb_delta_state_size(G, H, dim, vdim, taps), (long long)H * dim * vdim, ldz, G, H,  \
                        dim, vdim, taps, update_state};                                                               \
        return delta_prep_launch<T>(p, nt, B, s);                                                                     \
    }
TB_DELTA_PREP(f32, float)
TB_DELTA_PREP(bf16, __nv_bfloat16)

int tb_delta_scan(const float* qkv, const float* decay, const float* beta, const float* kq, float* state, float* out,
                  const int* seq_start, const int* slots, int B, int G, int H, int dim, int vdim, int taps,
                  cudaStream_t s) {
    DeltaScanArgs a{qkv, decay, beta, kq, state, out, seq_start, slots,
                    (long long)tb_delta_state_size(G, H, dim, vdim, taps), G, H, dim, vdim};
    return delta_scan_launch(a, B, s);
}
}

#include "tape.h"
TB_TAPE_REGISTER(tb_delta_prep_f32)
TB_TAPE_REGISTER(tb_delta_prep_bf16)
TB_TAPE_REGISTER(tb_delta_scan)
