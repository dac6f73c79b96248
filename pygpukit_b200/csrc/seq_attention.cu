// seq_attention.cu -- attention over a paged key/value cache for ragged batches (any mix of prompt portions and single
// decoded tokens), float32 arithmetic throughout.
//
// Cache: pages of PS positions; page p of a layer holds K rows [G][PS][D] and V rows [G][PS][Dv] in bfloat16 or float32;
// `table` [slots][max_pages] maps (sequence slot, position / PS) to a page.
//
//   mixer_prep:  per token, on the fused projection row [q | k | v | gate]: RMS norm of every query head (in place) and
//                key head (weights shared by the heads), optional value mixing v <- (1 - lam) v + lam v_first (or recording
//                v as v_first), K and V rows written to the cache at the token's position.
//   attention:   score = scale q.k -> cap tanh(score / cap) -> minus slope_h (i - j); key j is visible from query i when
//                j <= i and, with a chunk size C, floor(j / C) == floor(i / C); online softmax; P.V; optional output gate
//                out *= sigmoid(gate).  A block serves one tile of consecutive queries of one sequence and one KV head
//                (all query heads of its group), K/V tiles of 32 positions staged in shared memory, a lane per key.
#include "common.cuh"
#include "../../include/pgk_b200.h"

using namespace pgk;

namespace {

template <typename TC> __device__ __forceinline__ float cload(const TC* p);
template <> __device__ __forceinline__ float cload<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float cload<uint16_t>(const uint16_t* p) { return bf16_bits_to_f32(*p); }
template <typename TC> __device__ __forceinline__ void cstore(TC* p, float v);
template <> __device__ __forceinline__ void cstore<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void cstore<uint16_t>(uint16_t* p, float v) { *p = f32_to_bf16_bits(v); }

struct PrepArgs {
    float* proj; int ld;
    int H, G, D, Dv;
    const float* qw; const float* kw; float eps;
    int vmode; float lam; float* vfirst;            // 0: none, 1: record v, 2: mix with the recorded v
    void* kc; void* vc; const int* table; int max_pages, PS;
    const int* slot; const int* pos;
};

template <typename TC>
__global__ void __launch_bounds__(128) mixer_prep_kernel(PrepArgs a) {
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* row = a.proj + (size_t)t * a.ld;
    const int pos = a.pos[t], slot = a.slot[t];
    const int page = a.table[(size_t)slot * a.max_pages + pos / a.PS], r = pos % a.PS;
    const int koff = a.H * a.D, voff = koff + a.G * a.D;
    for (int u = warp; u < a.H + a.G; u += 4) {
        float* x = row + (size_t)u * a.D;            // query heads then key heads are contiguous
        float ss = 0.f;
        for (int d = lane; d < a.D; d += 32) ss = fmaf(x[d], x[d], ss);
        ss = warp_sum(ss);
        const float inv = 1.f / sqrtf(ss / (float)a.D + a.eps);
        if (u < a.H) {
            for (int d = lane; d < a.D; d += 32) x[d] = x[d] * inv * a.qw[d];
        } else {
            const int g = u - a.H;
            TC* dst = (TC*)a.kc + (((size_t)page * a.G + g) * a.PS + r) * a.D;
            for (int d = lane; d < a.D; d += 32) cstore<TC>(dst + d, x[d] * inv * a.kw[d]);
        }
    }
    const int GV = a.G * a.Dv;
    for (int i = threadIdx.x; i < GV; i += blockDim.x) {
        float v = row[voff + i];
        if (a.vmode == 1) a.vfirst[(size_t)t * GV + i] = v;
        else if (a.vmode == 2) v = (1.f - a.lam) * v + a.lam * a.vfirst[(size_t)t * GV + i];
        const int g = i / a.Dv, d = i - g * a.Dv;
        cstore<TC>((TC*)a.vc + (((size_t)page * a.G + g) * a.PS + r) * a.Dv + d, v);
    }
}

struct AttnArgs {
    const float* proj; int ld, q_off, g_off;
    float* out; int ldo;
    const void* kc; const void* vc; const int* table; int max_pages, PS;
    const int4* tiles;                  // (first token row, queries, slot, first position)
    const float* slopes;                // [H] or NULL
    int H, G, D, Dv, chunk, HB, gate;
    float scale, cap;
};

constexpr int KT = 32;                  // keys per tile = one per lane
constexpr int PPW = 4;                  // (query, head) pairs per warp
constexpr int NWARP = 8;

template <typename TC, int NV>
__global__ void __launch_bounds__(256) seq_attention_kernel(AttnArgs a) {
    extern __shared__ __align__(16) float sm[];
    const int D = a.D, Dv = a.Dv, DP = D + 1;
    float* qs = sm;                                   // [NWARP][D][PPW]
    float* Ks = qs + NWARP * D * PPW;                 // [KT][D + 1]
    float* Vs = Ks + KT * DP;                         // [KT][Dv]
    __shared__ long long krow[KT], vrow[KT];

    const int4 tile = a.tiles[blockIdx.x];
    const int t0 = tile.x, nq = tile.y, slot = tile.z, pos0 = tile.w;
    const int rep = a.H / a.G, hsplit = (rep + a.HB - 1) / a.HB;
    const int g = blockIdx.y / hsplit, hpart = blockIdx.y - g * hsplit;
    const int hb0 = g * rep + hpart * a.HB, nh = min(a.HB, rep - hpart * a.HB);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    // this warp's pairs
    int qi[PPW], hd[PPW], pi[PPW], lo[PPW];
    bool ok[PPW];
    float slope[PPW];
#pragma unroll
    for (int c = 0; c < PPW; ++c) {
        const int p = warp * PPW + c;
        qi[c] = p / a.HB;
        const int hh = p - qi[c] * a.HB;
        ok[c] = qi[c] < nq && hh < nh;
        hd[c] = hb0 + hh;
        pi[c] = pos0 + qi[c];
        lo[c] = a.chunk > 0 ? (pi[c] / a.chunk) * a.chunk : 0;
        slope[c] = (ok[c] && a.slopes) ? a.slopes[hd[c]] : 0.f;
    }
    for (int i = lane; i < D * PPW; i += 32) {
        const int d = i / PPW, c = i - d * PPW;
        float v = 0.f;
#pragma unroll
        for (int cc = 0; cc < PPW; ++cc)
            if (cc == c && ok[cc]) v = a.proj[(size_t)(t0 + qi[cc]) * a.ld + a.q_off + (size_t)hd[cc] * D + d];
        qs[(warp * D + d) * PPW + c] = v;
    }
    float m[PPW], l[PPW], acc[PPW][NV];
#pragma unroll
    for (int c = 0; c < PPW; ++c) {
        m[c] = -INFINITY; l[c] = 0.f;
#pragma unroll
        for (int v = 0; v < NV; ++v) acc[c][v] = 0.f;
    }
    const int jlo = a.chunk > 0 ? (pos0 / a.chunk) * a.chunk : 0, jhi = pos0 + nq - 1;
    const TC* kc = (const TC*)a.kc;
    const TC* vc = (const TC*)a.vc;
    for (int j0 = jlo; j0 <= jhi; j0 += KT) {
        __syncthreads();
        if (threadIdx.x < KT) {
            const int j = j0 + threadIdx.x;
            long long ko = -1, vo = -1;
            if (j <= jhi) {
                const int page = a.table[(size_t)slot * a.max_pages + j / a.PS], r = j % a.PS;
                ko = (((long long)page * a.G + g) * a.PS + r) * D;
                vo = (((long long)page * a.G + g) * a.PS + r) * Dv;
            }
            krow[threadIdx.x] = ko; vrow[threadIdx.x] = vo;
        }
        __syncthreads();
        for (int i = threadIdx.x; i < KT * D; i += blockDim.x) {
            const int r = i / D, d = i - r * D;
            Ks[r * DP + d] = krow[r] >= 0 ? cload<TC>(kc + krow[r] + d) : 0.f;
        }
        for (int i = threadIdx.x; i < KT * Dv; i += blockDim.x) {
            const int r = i / Dv, d = i - r * Dv;
            Vs[i] = vrow[r] >= 0 ? cload<TC>(vc + vrow[r] + d) : 0.f;
        }
        __syncthreads();
        // scores: lane = key
        float s[PPW] = {};
        const float* kr = Ks + lane * DP;
        const float4* q4 = (const float4*)(qs + warp * D * PPW);
        for (int d = 0; d < D; ++d) {
            const float kv = kr[d];
            const float4 q = q4[d];
            s[0] = fmaf(q.x, kv, s[0]); s[1] = fmaf(q.y, kv, s[1]);
            s[2] = fmaf(q.z, kv, s[2]); s[3] = fmaf(q.w, kv, s[3]);
        }
        const int j = j0 + lane;
        float p[PPW];
#pragma unroll
        for (int c = 0; c < PPW; ++c) {
            float sc = s[c] * a.scale;
            if (a.cap > 0.f) sc = a.cap * tanhf(sc / a.cap);
            sc -= slope[c] * (float)(pi[c] - j);
            const bool vis = ok[c] && j <= pi[c] && j >= lo[c];
            sc = vis ? sc : -INFINITY;
            const float mn = fmaxf(m[c], warp_max(sc));
            if (mn == -INFINITY) { p[c] = 0.f; continue; }      // uniform across the warp
            const float corr = expf(m[c] - mn);
            p[c] = expf(sc - mn);
            l[c] = l[c] * corr + warp_sum(p[c]);
            m[c] = mn;
#pragma unroll
            for (int v = 0; v < NV; ++v) acc[c][v] *= corr;
        }
        const int nvalid = min(KT, jhi - j0 + 1);
        for (int jj = 0; jj < nvalid; ++jj) {
            float pj[PPW];
#pragma unroll
            for (int c = 0; c < PPW; ++c) pj[c] = __shfl_sync(0xffffffffu, p[c], jj);
#pragma unroll
            for (int v = 0; v < NV; ++v) {
                const int dv = lane + 32 * v;
                const float vv = dv < Dv ? Vs[jj * Dv + dv] : 0.f;
#pragma unroll
                for (int c = 0; c < PPW; ++c) acc[c][v] = fmaf(pj[c], vv, acc[c][v]);
            }
        }
    }
#pragma unroll
    for (int c = 0; c < PPW; ++c) {
        if (!ok[c]) continue;
        const size_t t = t0 + qi[c];
        const float inv = l[c] > 0.f ? 1.f / l[c] : 0.f;
#pragma unroll
        for (int v = 0; v < NV; ++v) {
            const int dv = lane + 32 * v;
            if (dv >= Dv) continue;
            float o = acc[c][v] * inv;
            if (a.gate) {
                const float z = a.proj[t * a.ld + a.g_off + (size_t)hd[c] * Dv + dv];
                o *= 1.f / (1.f + expf(-z));
            }
            a.out[t * a.ldo + (size_t)hd[c] * Dv + dv] = o;
        }
    }
}

template <typename TC, int NV>
int launch_attn(const AttnArgs& a, int tiles, cudaStream_t st) {
    const size_t smem = sizeof(float) * ((size_t)NWARP * a.D * PPW + (size_t)KT * (a.D + 1) + (size_t)KT * a.Dv);
    PGK_REQUIRE(smem <= 200 * 1024, "seq_attention failed: head sizes %d / %d need %zu bytes of shared memory", a.D, a.Dv, smem);
    static size_t configured = 0;
    if (smem > 48 * 1024 && configured == 0) {
        PGK_CUDA(cudaFuncSetAttribute(seq_attention_kernel<TC, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        configured = 1;
    }
    const int rep = a.H / a.G, hsplit = (rep + a.HB - 1) / a.HB;
    PGK_CUDA(launch(seq_attention_kernel<TC, NV>, dim3(tiles, a.G * hsplit), dim3(256), smem, st, a));
    return 0;
}

template <typename TC>
int launch_attn_nv(const AttnArgs& a, int tiles, cudaStream_t st) {
    const int nv = (a.Dv + 31) / 32;
    if (nv <= 1) return launch_attn<TC, 1>(a, tiles, st);
    if (nv <= 2) return launch_attn<TC, 2>(a, tiles, st);
    if (nv <= 4) return launch_attn<TC, 4>(a, tiles, st);
    if (nv <= 8) return launch_attn<TC, 8>(a, tiles, st);
    set_error("seq_attention failed: value size %d exceeds 256", a.Dv);
    return 1;
}

}  // namespace

extern "C" {

int pgk_seq_heads_per_block(int heads, int kv_heads) {
    const int rep = kv_heads > 0 ? heads / kv_heads : 1;
    return rep < NWARP * PPW ? (rep > 0 ? rep : 1) : NWARP * PPW;
}
int pgk_seq_queries_per_tile(int heads, int kv_heads) { return (NWARP * PPW) / pgk_seq_heads_per_block(heads, kv_heads); }

int pgk_seq_mixer_prep(float* proj, int ld, int tokens, int heads, int kv_heads, int dim, int vdim, const float* q_weight,
                       const float* k_weight, float eps, int v_mode, float lam, float* v_first, void* k_cache, void* v_cache,
                       int cache_dtype, const int32_t* table, int max_pages, int page_size, const int32_t* slot,
                       const int32_t* pos, void* stream) {
    PGK_REQUIRE(cache_dtype == 0 || cache_dtype == 2, "seq_mixer_prep failed: the cache is float32 (0) or bfloat16 (2), got %d", cache_dtype);
    PGK_REQUIRE(heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && dim > 0 && vdim > 0, "seq_mixer_prep failed: invalid head layout");
    PGK_REQUIRE(v_mode == 0 || v_first, "seq_mixer_prep failed: value mixing needs the v_first buffer");
    if (tokens <= 0) return 0;
    PrepArgs a{proj, ld, heads, kv_heads, dim, vdim, q_weight, k_weight, eps, v_mode, lam, v_first, k_cache, v_cache, table,
               max_pages, page_size, slot, pos};
    if (cache_dtype == 2) PGK_CUDA(launch(mixer_prep_kernel<uint16_t>, dim3(tokens), dim3(128), 0, (cudaStream_t)stream, a));
    else PGK_CUDA(launch(mixer_prep_kernel<float>, dim3(tokens), dim3(128), 0, (cudaStream_t)stream, a));
    return 0;
}

int pgk_seq_attention(const float* proj, int ld, int q_off, int gate_off, float* out, int ldo, const void* k_cache,
                      const void* v_cache, int cache_dtype, const int32_t* table, int max_pages, int page_size,
                      const int32_t* tiles, int n_tiles, const float* slopes, int heads, int kv_heads, int dim, int vdim,
                      int chunk, float scale, float softcap, int gate, void* stream) {
    PGK_REQUIRE(cache_dtype == 0 || cache_dtype == 2, "seq_attention failed: the cache is float32 (0) or bfloat16 (2), got %d", cache_dtype);
    PGK_REQUIRE(heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && dim > 0 && vdim > 0, "seq_attention failed: invalid head layout");
    if (n_tiles <= 0) return 0;
    AttnArgs a{proj, ld, q_off, gate_off, out, ldo, k_cache, v_cache, table, max_pages, page_size, (const int4*)tiles, slopes,
               heads, kv_heads, dim, vdim, chunk, pgk_seq_heads_per_block(heads, kv_heads), gate, scale, softcap};
    if (cache_dtype == 2) return launch_attn_nv<uint16_t>(a, n_tiles, (cudaStream_t)stream);
    return launch_attn_nv<float>(a, n_tiles, (cudaStream_t)stream);
}

}  // extern "C"
