// seq_latent.cu -- the row-wise pieces of latent attention on the paged cache, float32 arithmetic.
//
// A latent-attention layer caches, per position, ONE row [c (rank) | r (rot)]: the normalised key/value latent and the
// rotated key part that all heads share.  Per head h the key is [Wuk_h c | r] and the value Wuv_h c; with
// q~_h = Wuk_h^T q_h the score q_h . (Wuk_h c) equals q~_h . c, and sum_j p_j (Wuv_h c_j) equals Wuv_h (sum_j p_j c_j), so the
// attention kernel runs with one key/value head of row size rank + rot whose values are the first `rank` elements of the
// key row, and the two per-head matrices are applied to the query before and to the output after it.
//
//   latent_prep:  per token, on the fused projection row [dq (q_rank) | dkv (rank + rot) | ...]: RMS norm of dq in place,
//                 RMS norm of the latent into the cache row, rotation of the shared key part into the cache row.
//   rope_heads:   rotates the `rot` tail of every query head and places it behind the head's absorbed query.
//
// Rotation: dimension 2i is paired with 2i + 1 (interleaved), angle = position * inv_freq[i]; the angle is formed and
// reduced to [-pi, pi] in double (positions reach thousands, where a float32 product has lost four digits), sine and cosine
// in float32.  Dimensions from `rot_dims` on pass unchanged.
#include "common.cuh"
#include "../../include/pgk_b200.h"

using namespace pgk;

namespace {

template <typename TC> __device__ __forceinline__ void cstore(TC* p, float v);
template <> __device__ __forceinline__ void cstore<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void cstore<uint16_t>(uint16_t* p, float v) { *p = f32_to_bf16_bits(v); }

__device__ __forceinline__ void angle_sincos(int pos, double inv_freq, float& sn, float& cs) {
    const double a = (double)pos * inv_freq;
    const double two_pi = 6.283185307179586476925286766559;
    const float r = (float)(a - two_pi * rint(a / two_pi));
    sincosf(r, &sn, &cs);
}

__device__ __forceinline__ float block_sum_256(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) s += red[i];
    return s;
}

struct LatentPrepArgs {
    float* proj; int ld;
    int q_rank, rank, rot, rot_dims, kv_off;
    const float* qw; const float* cw; float w_off, eps;
    const double* inv_freq;
    void* kc; const int* table; int max_pages, PS;
    const int* slot; const int* pos;
};

template <typename TC>
__global__ void __launch_bounds__(256) latent_prep_kernel(LatentPrepArgs a) {
    __shared__ float red[8];
    const int t = blockIdx.x;
    float* dq = a.proj + (size_t)t * a.ld;
    const float* dkv = dq + a.kv_off;
    float sq = 0.f, sc = 0.f;
    for (int i = threadIdx.x; i < a.q_rank; i += blockDim.x) sq = fmaf(dq[i], dq[i], sq);
    for (int i = threadIdx.x; i < a.rank; i += blockDim.x) sc = fmaf(dkv[i], dkv[i], sc);
    sq = block_sum_256(sq, red);
    sc = block_sum_256(sc, red);
    const float iq = a.q_rank > 0 ? 1.f / sqrtf(sq / (float)a.q_rank + a.eps) : 0.f;
    const float ic = 1.f / sqrtf(sc / (float)a.rank + a.eps);
    for (int i = threadIdx.x; i < a.q_rank; i += blockDim.x) dq[i] = dq[i] * iq * (a.w_off + a.qw[i]);
    const int pos = a.pos[t], slot = a.slot[t];
    const int page = a.table[(size_t)slot * a.max_pages + pos / a.PS], r = pos % a.PS;
    TC* dst = (TC*)a.kc + ((size_t)page * a.PS + r) * (a.rank + a.rot);
    for (int i = threadIdx.x; i < a.rank; i += blockDim.x) cstore<TC>(dst + i, dkv[i] * ic * (a.w_off + a.cw[i]));
    const float* kr = dkv + a.rank;
    for (int i = threadIdx.x; i < a.rot_dims / 2; i += blockDim.x) {
        float sn, cs;
        angle_sincos(pos, a.inv_freq[i], sn, cs);
        const float u = kr[2 * i], v = kr[2 * i + 1];
        cstore<TC>(dst + a.rank + 2 * i, u * cs - v * sn);
        cstore<TC>(dst + a.rank + 2 * i + 1, v * cs + u * sn);
    }
    for (int i = a.rot_dims + threadIdx.x; i < a.rot; i += blockDim.x) cstore<TC>(dst + a.rank + i, kr[i]);
}

struct RopeHeadsArgs {
    const float* src; int lds, src_head, src_off;     // head h's tail starts at src[t, h * src_head + src_off]
    float* dst; int ldd, dst_head, dst_off;
    int H, rot, rot_dims;
    const double* inv_freq; const int* pos;
};

__global__ void __launch_bounds__(256) rope_heads_kernel(RopeHeadsArgs a) {
    const int t = blockIdx.x, pos = a.pos[t];
    const int half = a.rot_dims / 2;
    for (int i = threadIdx.x; i < a.H * half; i += blockDim.x) {
        const int h = i / half, p = i - h * half;
        float sn, cs;
        angle_sincos(pos, a.inv_freq[p], sn, cs);
        const float* s = a.src + (size_t)t * a.lds + (size_t)h * a.src_head + a.src_off;
        float* d = a.dst + (size_t)t * a.ldd + (size_t)h * a.dst_head + a.dst_off;
        const float u = s[2 * p], v = s[2 * p + 1];
        d[2 * p] = u * cs - v * sn;
        d[2 * p + 1] = v * cs + u * sn;
    }
    const int rest = a.rot - a.rot_dims;
    for (int i = threadIdx.x; i < a.H * rest; i += blockDim.x) {
        const int h = i / rest, p = a.rot_dims + (i - h * rest);
        a.dst[(size_t)t * a.ldd + (size_t)h * a.dst_head + a.dst_off + p] = a.src[(size_t)t * a.lds + (size_t)h * a.src_head + a.src_off + p];
    }
}

}  // namespace

extern "C" {

int pgk_seq_latent_prep(float* proj, int ld, int tokens, int q_rank, int kv_off, int rank, int rot, int rot_dims,
                        const float* q_weight, const float* c_weight, float weight_offset, float eps, const double* inv_freq,
                        void* k_cache, int cache_dtype, const int32_t* table, int max_pages, int page_size,
                        const int32_t* slot, const int32_t* pos, void* stream) {
    PGK_REQUIRE(cache_dtype == 0 || cache_dtype == 2, "seq_latent_prep failed: the cache is float32 (0) or bfloat16 (2), got %d", cache_dtype);
    PGK_REQUIRE(rank > 0 && rot >= 0 && rot_dims >= 0 && rot_dims <= rot && rot_dims % 2 == 0 && q_rank >= 0,
                "seq_latent_prep failed: rank %d, rotated part %d of which %d turn", rank, rot, rot_dims);
    if (tokens <= 0) return 0;
    LatentPrepArgs a{proj, ld, q_rank, rank, rot, rot_dims, kv_off, q_weight, c_weight, weight_offset, eps, inv_freq, k_cache,
                     table, max_pages, page_size, slot, pos};
    if (cache_dtype == 2) PGK_CUDA(launch(latent_prep_kernel<uint16_t>, dim3(tokens), dim3(256), 0, (cudaStream_t)stream, a));
    else PGK_CUDA(launch(latent_prep_kernel<float>, dim3(tokens), dim3(256), 0, (cudaStream_t)stream, a));
    return 0;
}

int pgk_seq_rope_heads(const float* src, int lds, int src_head, int src_off, float* dst, int ldd, int dst_head, int dst_off,
                       int tokens, int heads, int rot, int rot_dims, const double* inv_freq, const int32_t* pos, void* stream) {
    PGK_REQUIRE(heads > 0 && rot >= 0 && rot_dims >= 0 && rot_dims <= rot && rot_dims % 2 == 0,
                "seq_rope_heads failed: %d heads, rotated part %d of which %d turn", heads, rot, rot_dims);
    if (tokens <= 0 || rot == 0) return 0;
    RopeHeadsArgs a{src, lds, src_head, src_off, dst, ldd, dst_head, dst_off, heads, rot, rot_dims, inv_freq, pos};
    PGK_CUDA(launch(rope_heads_kernel, dim3(tokens), dim3(256), 0, (cudaStream_t)stream, a));
    return 0;
}

}  // extern "C"
