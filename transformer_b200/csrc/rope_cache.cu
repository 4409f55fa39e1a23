// Rotary position encoding of q and k, fused with the write of k and v into the paged cache.
//
// qkv is [nt, (nh + 2 nkvh) dh] with the heads ordered q, k, v
// (models/llama/common/src/compute.rs:225-227).  q is rotated in place; k is rotated and stored,
// v is copied, into the page that holds the token's position
// (the reference stores k, v at pos..pos+seq of the request's cache, compute.rs:244-263).
// Angles come from a float table [positions, dh/2] built on the host in double precision:
// angle(p, i) = p * theta^(-2i/dh).
//
// Cache of one layer: K and V each [pages, nkvh, TB_PAGE, dh].
#include "common.cuh"

#define ROPE_HEADS 4   // heads per block when there are few tokens; 32 (a full block of 16-byte items) for prompts

template <typename T>
__global__ void rope_cache_kernel(T* __restrict__ qkv, const int* __restrict__ tok_seq,
                                  const int* __restrict__ tok_pos, const int* __restrict__ page_table,
                                  int max_pages, const float* __restrict__ cos_t,
                                  const float* __restrict__ sin_t, T* __restrict__ kc, T* __restrict__ vc,
                                  int nh, int nkvh, int dh, int half_pairing, int hpb) {
    pdl_sync();
    // grid: (token, chunk of hpb heads out of q heads, k heads, v heads in that order)
    const int t = blockIdx.x;
    const int head_lo = blockIdx.y * hpb;
    const int head_hi = min(head_lo + hpb, nh + 2 * nkvh);
    const int pos = tok_pos[t];
    const int half = dh >> 1;
    T* row = qkv + (size_t)t * (nh + 2 * nkvh) * dh;
    const float* cs = cos_t + (size_t)pos * half;
    const float* sn = sin_t + (size_t)pos * half;
    size_t cache_row = 0;
    if (kc) {
        const int page = page_table[(size_t)tok_seq[t] * max_pages + pos / TB_PAGE];
        cache_row = ((size_t)page * nkvh * TB_PAGE + (pos % TB_PAGE)) * dh;  // + g * TB_PAGE * dh
    }
    const int rot_hi = min(head_hi, nh + nkvh);
    for (int idx = threadIdx.x; idx < (rot_hi - head_lo) * half; idx += blockDim.x) {
        const int head = head_lo + idx / half, i = idx % half;
        const int i0 = half_pairing ? i : 2 * i;
        const int i1 = half_pairing ? i + half : 2 * i + 1;
        T* h = row + (size_t)head * dh;
        const float x0 = ldf(h + i0), x1 = ldf(h + i1);
        const float c = cs[i], s = sn[i];
        const float y0 = x0 * c - x1 * s;
        const float y1 = x0 * s + x1 * c;
        if (head < nh) {
            stf(h + i0, y0);
            stf(h + i1, y1);
        } else if (kc) {
            T* dst = kc + cache_row + (size_t)(head - nh) * TB_PAGE * dh;
            stf(dst + i0, y0);
            stf(dst + i1, y1);
        }
    }
    if (vc && head_hi > nh + nkvh) {
        const int v_lo = max(head_lo, nh + nkvh);
        for (int idx = threadIdx.x; idx < (head_hi - v_lo) * dh; idx += blockDim.x) {
            const int head = v_lo + idx / dh, c = idx % dh;
            vc[cache_row + (size_t)(head - nh - nkvh) * TB_PAGE * dh + c] = row[(size_t)head * dh + c];
        }
    }
}

// The same with 8 values per thread and 16-byte accesses (head sizes that are a multiple of 16).  EARLY (a few
// tokens: decoding) reads the angles before the dependency wait; with many tokens the kernel is bound by memory
// traffic and does better with the registers that would cost.
template <typename T, bool EARLY>
__global__ void rope_cache_vec_kernel(T* __restrict__ qkv, const int* __restrict__ tok_seq,
                                      const int* __restrict__ tok_pos, const int* __restrict__ page_table,
                                      int max_pages, const float* __restrict__ cos_t,
                                      const float* __restrict__ sin_t, T* __restrict__ kc, T* __restrict__ vc,
                                      int nh, int nkvh, int dh, int half_pairing, int hpb) {
    // Positions and the angle table were there before the step began: the angles of this thread's first item are
    // read before the wait for the kernel that wrote q, k and v (the table is touched once per layer and has
    // left L2 since the last step).
    const int t = blockIdx.x;
    const int head_lo = blockIdx.y * hpb;
    const int head_hi = min(head_lo + hpb, nh + 2 * nkvh);
    const int pos = tok_pos[t];
    const int half = dh >> 1;
    T* row = qkv + (size_t)t * (nh + 2 * nkvh) * dh;
    const float* cs = cos_t + (size_t)pos * half;
    const float* sn = sin_t + (size_t)pos * half;
    float c0[8], s0[8];
    if (EARLY) {
        const int u = threadIdx.x % (dh / 16);
        load8(cs + u * 8, c0);
        load8(sn + u * 8, s0);
    }
    size_t cache_row = 0;
    if (kc) {
        const int page = page_table[(size_t)tok_seq[t] * max_pages + pos / TB_PAGE];
        cache_row = ((size_t)page * nkvh * TB_PAGE + (pos % TB_PAGE)) * dh;
    }
    pdl_sync();
    const int rot_hi = min(head_hi, nh + nkvh);
    const int units = dh / 16;                 // work items per head: 16 values = 8 pairs each
    for (int idx = threadIdx.x; idx < (rot_hi - head_lo) * units; idx += blockDim.x) {
        const int head = head_lo + idx / units, u = idx % units;
        T* h = row + (size_t)head * dh;
        T* dst = head < nh ? h : (kc ? kc + cache_row + (size_t)(head - nh) * TB_PAGE * dh : nullptr);
        float a[8], b[8], c[8], s[8], ya[8], yb[8];
        if (EARLY && idx == (int)threadIdx.x) {   // the item whose angles are in registers already
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                c[e] = c0[e];
                s[e] = s0[e];
            }
        } else {
            load8(cs + u * 8, c);              // pairs 8u .. 8u+7
            load8(sn + u * 8, s);
        }
        if (half_pairing) {                    // pair i = (x[i], x[i + half])
            load8(h + u * 8, a);
            load8(h + half + u * 8, b);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                ya[e] = a[e] * c[e] - b[e] * s[e];
                yb[e] = a[e] * s[e] + b[e] * c[e];
            }
            if (dst) {
                store8(dst + u * 8, ya);
                store8(dst + half + u * 8, yb);
            }
        } else {                               // pair i = (x[2i], x[2i+1]): 16 consecutive values
            load8(h + u * 16, a);
            load8(h + u * 16 + 8, b);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                ya[2 * e] = a[2 * e] * c[e] - a[2 * e + 1] * s[e];
                ya[2 * e + 1] = a[2 * e] * s[e] + a[2 * e + 1] * c[e];
                yb[2 * e] = b[2 * e] * c[4 + e] - b[2 * e + 1] * s[4 + e];
                yb[2 * e + 1] = b[2 * e] * s[4 + e] + b[2 * e + 1] * c[4 + e];
            }
            if (dst) {
                store8(dst + u * 16, ya);
                store8(dst + u * 16 + 8, yb);
            }
        }
    }
    if (vc && head_hi > nh + nkvh) {
        const int v_lo = max(head_lo, nh + nkvh);
        const int per = dh / 8;
        for (int idx = threadIdx.x; idx < (head_hi - v_lo) * per; idx += blockDim.x) {
            const int head = v_lo + idx / per, c8 = (idx % per) * 8;
            float f[8];
            load8(row + (size_t)head * dh + c8, f);
            store8(vc + cache_row + (size_t)(head - nh - nkvh) * TB_PAGE * dh + c8, f);
        }
    }
}

template <typename T>
static int rope_cache_launch(void* qkv, const int* tok_seq, const int* tok_pos, const int* page_table,
                             int max_pages, const float* cos_t, const float* sin_t, void* kc, void* vc,
                             int nt, int nh, int nkvh, int dh, int half_pairing, cudaStream_t s) {
    if (nt < 0 || nh <= 0 || nkvh <= 0 || dh <= 0 || (dh & 1)) return TB_ERR_ARG;
    if ((kc == nullptr) != (vc == nullptr)) return TB_ERR_ARG;
    if (nt == 0) return 0;
    // few tokens (decoding): many small blocks, so that every SM has some; prompts: blocks of 256 full threads
    const int hpb = nt >= 256 ? 8 * ROPE_HEADS : ROPE_HEADS;
    dim3 grid(nt, (nh + 2 * nkvh + hpb - 1) / hpb);
    if (dh % 16 == 0 && (((uintptr_t)qkv | (uintptr_t)kc | (uintptr_t)vc) & 15) == 0) {
        int threads = (hpb * (dh / 16) + 31) / 32 * 32;
        threads = threads < 64 ? 64 : threads > 256 ? 256 : threads;
        if (nt < 256)
            TB_LAUNCH((rope_cache_vec_kernel<T, true>), grid, threads, 0, s, (T*)qkv, tok_seq, tok_pos, page_table,
                      max_pages, cos_t, sin_t, (T*)kc, (T*)vc, nh, nkvh, dh, half_pairing, hpb);
        else
            TB_LAUNCH((rope_cache_vec_kernel<T, false>), grid, threads, 0, s, (T*)qkv, tok_seq, tok_pos, page_table,
                      max_pages, cos_t, sin_t, (T*)kc, (T*)vc, nh, nkvh, dh, half_pairing, hpb);
        return tb_last_error();
    }
    TB_LAUNCH((rope_cache_kernel<T>), grid, nt >= 256 ? 256 : 128, 0, s, (T*)qkv, tok_seq, tok_pos, page_table, max_pages,
              cos_t, sin_t, (T*)kc, (T*)vc, nh, nkvh, dh, half_pairing, hpb);
    return tb_last_error();
}

// The same step for a mixer that norms its whole query and key projections first and rotates only a part of every
// head, with value heads of a size of their own.  Row of z: q (nh dk) | k (nkvh dk) | v (nkvh dv) | ...
//   q <- q / sqrt(mean over ALL nh dk entries (q^2) + eps) * q_norm,   k alike over its nkvh dk entries;
//   the first rdims entries of every head turn by the token's angles (table [positions, rdims / 2]), the rest pass;
//   q is written back in place, k and v go to the cache:  K [pages, nkvh, TB_PAGE, dk],  V [pages, nkvh, TB_PAGE, dv].
// Statistics, the norm and the rotation are float; one rounding at each store.  A block per token.
template <typename T>
__global__ void __launch_bounds__(256)
qknorm_rope_cache_kernel(T* __restrict__ z, int ldz, const float* __restrict__ q_norm, const float* __restrict__ k_norm,
                         float eps, const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                         const int* __restrict__ page_table, int max_pages, const float* __restrict__ cos_t,
                         const float* __restrict__ sin_t, T* __restrict__ kc, T* __restrict__ vc, int nh, int nkvh,
                         int dk, int dv, int rdims, int half_pairing) {
    pdl_sync();
    __shared__ float red[33];
    const int t = blockIdx.x;
    const int pos = tok_pos[t];
    const int nq = nh * dk, nk = nkvh * dk;
    T* row = z + (size_t)t * ldz;
    float rq = 1.f, rk = 1.f;
    if (q_norm) {
        float ss = 0.f;
        for (int c = threadIdx.x; c < nq; c += blockDim.x) {
            const float x = ldf(row + c);
            ss += x * x;
        }
        rq = 1.0f / sqrtf(block_sum(ss, red) / (float)nq + eps);
    }
    if (k_norm) {
        float ss = 0.f;
        for (int c = threadIdx.x; c < nk; c += blockDim.x) {
            const float x = ldf(row + nq + c);
            ss += x * x;
        }
        rk = 1.0f / sqrtf(block_sum(ss, red) / (float)nk + eps);
    }
    const int rp = rdims >> 1;                  // rotated pairs per head
    const float* cs = cos_t + (size_t)pos * rp;
    const float* sn = sin_t + (size_t)pos * rp;
    size_t cache_row = 0;
    if (kc) {
        const int page = page_table[(size_t)tok_seq[t] * max_pages + pos / TB_PAGE];
        cache_row = (size_t)page * nkvh * TB_PAGE + (pos % TB_PAGE);      // + head * TB_PAGE, times the head size
    }
    // rotated pairs of the query heads, then of the key heads
    for (int idx = threadIdx.x; idx < (nh + nkvh) * rp; idx += blockDim.x) {
        const int head = idx / rp, i = idx - head * rp;
        const int i0 = half_pairing ? i : 2 * i, i1 = half_pairing ? i + rp : 2 * i + 1;
        const bool is_q = head < nh;
        const int base = head * dk;             // column of the head's first entry in the row (q and k are adjacent)
        const float* w = is_q ? q_norm : k_norm;
        const int wb = is_q ? base : base - nq;
        const float r = is_q ? rq : rk;
        const float x0 = ldf(row + base + i0) * r * (w ? w[wb + i0] : 1.f);
        const float x1 = ldf(row + base + i1) * r * (w ? w[wb + i1] : 1.f);
        const float c = cs[i], s = sn[i];
        const float y0 = x0 * c - x1 * s, y1 = x1 * c + x0 * s;
        if (is_q) {
            stf(row + base + i0, y0);
            stf(row + base + i1, y1);
        } else if (kc) {
            T* dst = kc + (cache_row + (size_t)(head - nh) * TB_PAGE) * dk;
            stf(dst + i0, y0);
            stf(dst + i1, y1);
        }
    }
    // the entries that pass
    const int rest = dk - rdims;
    for (int idx = threadIdx.x; idx < (nh + nkvh) * rest; idx += blockDim.x) {
        const int head = idx / rest, c = rdims + idx - head * rest;
        const bool is_q = head < nh;
        const int base = head * dk;
        const float* w = is_q ? q_norm : k_norm;
        const float y = ldf(row + base + c) * (is_q ? rq : rk) * (w ? w[(is_q ? base : base - nq) + c] : 1.f);
        if (is_q) stf(row + base + c, y);
        else if (kc) stf(kc + (cache_row + (size_t)(head - nh) * TB_PAGE) * dk + c, y);
    }
    if (vc)
        for (int idx = threadIdx.x; idx < nkvh * dv; idx += blockDim.x) {
            const int head = idx / dv, c = idx - head * dv;
            vc[(cache_row + (size_t)head * TB_PAGE) * dv + c] = row[nq + nk + idx];
        }
}

// The same, eight entries at a time with 16-byte accesses: head sizes, the rotated part and the row pitch multiples
// of eight, adjacent pairs.
template <typename T>
__global__ void __launch_bounds__(256)
qknorm_rope_cache_vec_kernel(T* __restrict__ z, int ldz, const float* __restrict__ q_norm,
                             const float* __restrict__ k_norm, float eps, const int* __restrict__ tok_seq,
                             const int* __restrict__ tok_pos, const int* __restrict__ page_table, int max_pages,
                             const float* __restrict__ cos_t, const float* __restrict__ sin_t, T* __restrict__ kc,
                             T* __restrict__ vc, int nh, int nkvh, int dk, int dv, int rdims) {
    pdl_sync();
    __shared__ float red[33];
    const int t = blockIdx.x;
    const int pos = tok_pos[t];
    const int nq = nh * dk, nk = nkvh * dk;
    T* row = z + (size_t)t * ldz;
    float rq = 1.f, rk = 1.f;
    if (q_norm) {
        float ss = 0.f;
        for (int c = threadIdx.x * 8; c < nq; c += blockDim.x * 8) {
            float x[8];
            load8(row + c, x);
#pragma unroll
            for (int e = 0; e < 8; ++e) ss += x[e] * x[e];
        }
        rq = 1.0f / sqrtf(block_sum(ss, red) / (float)nq + eps);
    }
    if (k_norm) {
        float ss = 0.f;
        for (int c = threadIdx.x * 8; c < nk; c += blockDim.x * 8) {
            float x[8];
            load8(row + nq + c, x);
#pragma unroll
            for (int e = 0; e < 8; ++e) ss += x[e] * x[e];
        }
        rk = 1.0f / sqrtf(block_sum(ss, red) / (float)nk + eps);
    }
    const int rp = rdims >> 1;
    const float* cs = cos_t + (size_t)pos * rp;
    const float* sn = sin_t + (size_t)pos * rp;
    size_t cache_row = 0;
    if (kc) {
        const int page = page_table[(size_t)tok_seq[t] * max_pages + pos / TB_PAGE];
        cache_row = (size_t)page * nkvh * TB_PAGE + (pos % TB_PAGE);
    }
    for (int c = threadIdx.x * 8; c < nq + nk; c += blockDim.x * 8) {
        const bool is_q = c < nq;
        const int head = c / dk, within = c - head * dk;          // q and k heads are adjacent and equally wide
        const float* w = is_q ? q_norm : k_norm;
        const float r = is_q ? rq : rk;
        float x[8], y[8];
        load8(row + c, x);
        if (w) {
            float wv[8];
            load8(w + (is_q ? c : c - nq), wv);
#pragma unroll
            for (int e = 0; e < 8; ++e) x[e] *= r * wv[e];
        }
        if (within < rdims) {           // four pairs, angles within / 2 .. within / 2 + 3
            const float4 c4 = *reinterpret_cast<const float4*>(cs + (within >> 1));
            const float4 s4 = *reinterpret_cast<const float4*>(sn + (within >> 1));
            const float cc[4] = {c4.x, c4.y, c4.z, c4.w}, ss[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                y[2 * e] = x[2 * e] * cc[e] - x[2 * e + 1] * ss[e];
                y[2 * e + 1] = x[2 * e + 1] * cc[e] + x[2 * e] * ss[e];
            }
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) y[e] = x[e];
        }
        if (is_q) store8(row + c, y);
        else if (kc) store8(kc + (cache_row + (size_t)(head - nh) * TB_PAGE) * dk + within, y);
    }
    if (vc)
        for (int c = threadIdx.x * 8; c < nkvh * dv; c += blockDim.x * 8) {
            const int head = c / dv, within = c - head * dv;
            float x[8];
            load8(row + nq + nk + c, x);
            store8(vc + (cache_row + (size_t)head * TB_PAGE) * dv + within, x);
        }
}

template <typename T>
static int qknorm_rope_cache_launch(void* z, int ldz, const float* q_norm, const float* k_norm, float eps,
                                    const int* tok_seq, const int* tok_pos, const int* page_table, int max_pages,
                                    const float* cos_t, const float* sin_t, void* kc, void* vc, int nt, int nh,
                                    int nkvh, int dk, int dv, int rdims, int half_pairing, cudaStream_t s) {
    if (nt < 0 || nh <= 0 || nkvh <= 0 || dk <= 0 || dv <= 0 || rdims < 0 || rdims > dk || (rdims & 1)) return TB_ERR_ARG;
    if ((kc == nullptr) != (vc == nullptr) || ldz < (nh + nkvh) * dk + nkvh * dv) return TB_ERR_ARG;
    if (nt == 0) return 0;
    if (!half_pairing && dk % 8 == 0 && dv % 8 == 0 && rdims % 8 == 0 && ldz % 8 == 0 &&
        (((uintptr_t)z | (uintptr_t)kc | (uintptr_t)vc | (uintptr_t)q_norm | (uintptr_t)k_norm | (uintptr_t)cos_t |
          (uintptr_t)sin_t) & 15) == 0) {
        TB_LAUNCH((qknorm_rope_cache_vec_kernel<T>), nt, 256, 0, s, (T*)z, ldz, q_norm, k_norm, eps, tok_seq, tok_pos,
                  page_table, max_pages, cos_t, sin_t, (T*)kc, (T*)vc, nh, nkvh, dk, dv, rdims);
        return tb_last_error();
    }
    TB_LAUNCH((qknorm_rope_cache_kernel<T>), nt, 256, 0, s, (T*)z, ldz, q_norm, k_norm, eps, tok_seq, tok_pos, page_table,
              max_pages, cos_t, sin_t, (T*)kc, (T*)vc, nh, nkvh, dk, dv, rdims, half_pairing);
    return tb_last_error();
}

extern "C" {
int tb_rope_cache_f32(void* qkv, const int* tok_seq, const int* tok_pos, const int* page_table, int max_pages,
                      const float* cos_t, const float* sin_t, void* kc, void* vc, int nt, int nh, int nkvh,
                      int dh, int half_pairing, cudaStream_t s) {
    return rope_cache_launch<float>(qkv, tok_seq, tok_pos, page_table, max_pages, cos_t, sin_t, kc, vc, nt, nh,
                                    nkvh, dh, half_pairing, s);
}
int tb_rope_cache_bf16(void* qkv, const int* tok_seq, const int* tok_pos, const int* page_table, int max_pages,
                       const float* cos_t, const float* sin_t, void* kc, void* vc, int nt, int nh, int nkvh,
                       int dh, int half_pairing, cudaStream_t s) {
    return rope_cache_launch<__nv_bfloat16>(qkv, tok_seq, tok_pos, page_table, max_pages, cos_t, sin_t, kc, vc,
                                            nt, nh, nkvh, dh, half_pairing, s);
}
#define TB_QKNORM_ROPE(NAME, T)                                                                                        \
    int NAME(void* z, int ldz, const float* q_norm, const float* k_norm, float eps, const int* tok_seq,               \
             const int* tok_pos, const int* page_table, int max_pages, const float* cos_t, const float* sin_t,        \
             void* kc, void* vc, int nt, int nh, int nkvh, int dk, int dv, int rdims, int half_pairing,               \
             cudaStream_t s) {                                                                                        \
        return qknorm_rope_cache_launch<T>(z, ldz, q_norm, k_norm, eps, tok_seq, tok_pos, page_table, max_pages,      \
                                           cos_t, sin_t, kc, vc, nt, nh, nkvh, dk, dv, rdims, half_pairing, s);       \
    }
TB_QKNORM_ROPE(tb_qknorm_rope_cache_f32, float)
TB_QKNORM_ROPE(tb_qknorm_rope_cache_bf16, __nv_bfloat16)
}

// replayable from C++ (tape.h)
#include "tape.h"
TB_TAPE_REGISTER(tb_rope_cache_f32)
TB_TAPE_REGISTER(tb_rope_cache_bf16)
TB_TAPE_REGISTER(tb_qknorm_rope_cache_f32)
TB_TAPE_REGISTER(tb_qknorm_rope_cache_bf16)
