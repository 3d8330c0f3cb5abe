// Paged attention, row form with shared key tiles: one block per (query row, key/value head, group of query heads).
// The block brings tiles of 32 keys (and their values) into shared memory once and every warp of the block works on
// query heads of its own over them, so the heads of a group read their keys once and no results of different warps
// have to be merged. All arithmetic is 32-bit, also where the cache is bfloat16; queries are 32-bit or bfloat16.
//
// What a row sees and how a score is made are parameters:
//   window   w > 0: the query at position P sees keys P-w+1 .. P
//   chunk    c > 0: only keys of the query's own block of c positions counted from 0, floor(j / c) = floor(P / c)
//   slopes   [H] or null: slope_h * (P - j) is taken off the score of key j (a bias that grows with the distance)
//   sinks    [H] or null: the softmax's denominator also holds exp(sinks_h), a term without key or value
//   values   a width ``vd`` of their own; they may lie in pages of their own or be the first vd columns of the key
//            rows (``v_row`` is the length of the rows they lie in), which serves attention over a shared latent whose
//            keys are [latent, rotated part] and whose values are the latent itself
// The online softmax walks the keys in tiles counted from the row's first visible key, so a row's result depends on
// that row's query, position and cache contents only.
#include "common.cuh"

namespace gi {

constexpr int kRowsTile = 32;        // keys per tile: one per lane

template <typename T> struct Pair2;
template <> struct Pair2<float> {
    static __device__ __forceinline__ float2 load(const float* p) { return *reinterpret_cast<const float2*>(p); }
};
template <> struct Pair2<__nv_bfloat16> {
    static __device__ __forceinline__ float2 load(const __nv_bfloat16* p) {
        return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
    }
};

struct RowsArgs {
    const void* q; int q_is_f32; int ldq;          // queries [T, ldq], head h at column h * hd
    const void* k_cache; const void* v_cache;      // [pages, Hkv, page_size, hd] and [pages, Hkv, page_size, v_row]
    void* out; int out_is_f32; int ldo;            // [T, ldo], head h at column h * vd
    const int* row_req; const int* positions; const int* block_tables; int table_stride;
    int H, Hkv, hd, vd, v_row, page_size;
    float scale; int window, chunk;
    const float* slopes; const float* sinks;
    int heads_per_block;                           // query heads of one key/value head that a block takes
    int ks;                                        // row length of the key tile in shared memory (elements)
    int alias;                                     // the values are the first vd columns of the key rows
};

// HPW: query heads per warp; VI: value dimensions per lane (vd <= 32 * VI).
template <typename T, int HPW, int VI>
__global__ void __launch_bounds__(128)
attention_rows_kernel(const RowsArgs a) {
    pdl_prologue();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int t = blockIdx.x, g = blockIdx.y;
    const int group = a.H / a.Hkv;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int hdp = (a.hd + 1) & ~1;
    const int first_head = blockIdx.z * a.heads_per_block;        // within the group
    const int n_heads = min(a.heads_per_block, group - first_head);

    float* s_q = reinterpret_cast<float*>(smem_raw);                              // [heads_per_block][hdp]
    T* s_k = reinterpret_cast<T*>(s_q + a.heads_per_block * hdp);                  // [32][ks]
    T* s_v = a.alias ? s_k : s_k + kRowsTile * a.ks;                               // [32][vd]
    const int vs = a.alias ? a.ks : a.vd;

    const int pos = a.positions[t];
    int lo = 0;
    if (a.window > 0) lo = max(lo, pos - a.window + 1);
    if (a.chunk > 0) lo = max(lo, pos / a.chunk * a.chunk);
    const int* table = a.block_tables + static_cast<size_t>(a.row_req[t]) * a.table_stride;

    // the block's queries, 32-bit; an odd head size is padded with a zero
    for (int i = threadIdx.x; i < n_heads * hdp; i += blockDim.x) {
        const int hh = i / hdp, d = i % hdp;
        float v = 0.f;
        if (d < a.hd) {
            const size_t off = static_cast<size_t>(t) * a.ldq + static_cast<size_t>(g * group + first_head + hh) * a.hd + d;
            v = a.q_is_f32 ? static_cast<const float*>(a.q)[off] : to_float(static_cast<const __nv_bfloat16*>(a.q)[off]);
        }
        s_q[i] = v;
    }

    float acc[HPW][VI];
    float m[HPW], l[HPW], slope[HPW];
#pragma unroll
    for (int hh = 0; hh < HPW; ++hh) {
        m[hh] = -INFINITY; l[hh] = 0.f;
        const int head = first_head + warp * HPW + hh;
        slope[hh] = (a.slopes && head < group) ? a.slopes[g * group + head] : 0.f;
#pragma unroll
        for (int i = 0; i < VI; ++i) acc[hh][i] = 0.f;
    }
    const bool warp_active = warp * HPW < n_heads;
    const T* kc = static_cast<const T*>(a.k_cache);
    const T* vc = static_cast<const T*>(a.v_cache);

    for (int base = lo; base <= pos; base += kRowsTile) {
        const int n_keys = min(kRowsTile, pos - base + 1);
        __syncthreads();                       // the tile before is done with (and the queries are written)
        // every warp fetches keys of its own: key j of the tile lands in row j
        for (int j = warp; j < n_keys; j += blockDim.x >> 5) {
            const int p = base + j;
            const int page = table[p / a.page_size];
            const size_t row = (static_cast<size_t>(page) * a.Hkv + g) * a.page_size + (p % a.page_size);
            const T* src = kc + row * a.hd;
            T* dst = s_k + j * a.ks;
            for (int d = lane; d < hdp; d += 32) dst[d] = d < a.hd ? src[d] : from_float<T>(0.f);
            if (!a.alias) {
                const T* vsrc = vc + row * a.v_row;
                T* vdst = s_v + j * a.vd;
                for (int d = lane; d < a.vd; d += 32) vdst[d] = vsrc[d];
            }
        }
        __syncthreads();
        if (!warp_active) continue;
        // scores: a lane per key, the block's heads one after the other over the same key row
        float s[HPW];
#pragma unroll
        for (int hh = 0; hh < HPW; ++hh) s[hh] = 0.f;
        const bool valid = lane < n_keys;
        if (valid) {
            const T* krow = s_k + lane * a.ks;
            for (int d = 0; d < hdp; d += 2) {
                const float2 kk = Pair2<T>::load(krow + d);
#pragma unroll
                for (int hh = 0; hh < HPW; ++hh) {
                    const float2 qq = *reinterpret_cast<const float2*>(s_q + (warp * HPW + hh) * hdp + d);
                    s[hh] = fmaf(qq.x, kk.x, s[hh]);
                    s[hh] = fmaf(qq.y, kk.y, s[hh]);
                }
            }
        }
        float p[HPW];
#pragma unroll
        for (int hh = 0; hh < HPW; ++hh) {
            const float score = valid ? s[hh] * a.scale - slope[hh] * static_cast<float>(pos - (base + lane)) : -INFINITY;
            const float m_new = fmaxf(m[hh], warp_max(score));          // finite: a tile always holds a visible key
            p[hh] = valid ? expf(score - m_new) : 0.f;
            const float corr = (m[hh] == -INFINITY) ? 0.f : expf(m[hh] - m_new);
            l[hh] = l[hh] * corr + warp_sum(p[hh]);
#pragma unroll
            for (int i = 0; i < VI; ++i) acc[hh][i] *= corr;
            m[hh] = m_new;
        }
        for (int j = 0; j < n_keys; ++j) {
            float pj[HPW];
#pragma unroll
            for (int hh = 0; hh < HPW; ++hh) pj[hh] = __shfl_sync(0xffffffffu, p[hh], j);
            const T* vrow = s_v + j * vs;
#pragma unroll
            for (int i = 0; i < VI; ++i) {
                const int d = lane + 32 * i;
                if (d < a.vd) {
                    const float v = to_float(vrow[d]);
#pragma unroll
                    for (int hh = 0; hh < HPW; ++hh) acc[hh][i] = fmaf(pj[hh], v, acc[hh][i]);
                }
            }
        }
    }

    if (!warp_active) return;
#pragma unroll
    for (int hh = 0; hh < HPW; ++hh) {
        const int head = first_head + warp * HPW + hh;
        if (head >= group) continue;
        const int h = g * group + head;
        float M = m[hh], L = l[hh], f = 1.f;
        if (a.sinks) {
            const float sk = a.sinks[h];
            M = fmaxf(M, sk);
            f = expf(m[hh] - M);
            L = L * f + expf(sk - M);
        }
        const float mul = f / L;
        const size_t o = static_cast<size_t>(t) * a.ldo + static_cast<size_t>(h) * a.vd;
#pragma unroll
        for (int i = 0; i < VI; ++i) {
            const int d = lane + 32 * i;
            if (d < a.vd) {
                const float v = acc[hh][i] * mul;
                if (a.out_is_f32) static_cast<float*>(a.out)[o + d] = v;
                else static_cast<__nv_bfloat16*>(a.out)[o + d] = __float2bfloat16_rn(v);
            }
        }
    }
}

constexpr int kRowsMaxValueDim = 512;
constexpr int kRowsMaxHeadDim = 1024;

template <typename T, int HPW, int VI>
static int launch_rows(const RowsArgs& a, int T_rows, int blocks_z, int warps, size_t smem, cudaStream_t st) {
    auto kernel = attention_rows_kernel<T, HPW, VI>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) { set_error("attention_rows: %s", cudaGetErrorString(e)); return 1; }
    }
    launch_kernel(kernel, dim3(T_rows, a.Hkv, blocks_z), dim3(warps * 32), smem, st, a);
    return check_launch("attention_rows");
}

template <typename T, int HPW>
static int launch_rows_vi(const RowsArgs& a, int T_rows, int blocks_z, int warps, size_t smem, cudaStream_t st) {
    if (a.vd <= 128) return launch_rows<T, HPW, 4>(a, T_rows, blocks_z, warps, smem, st);
    if (a.vd <= 256) return launch_rows<T, HPW, 8>(a, T_rows, blocks_z, warps, smem, st);
    return launch_rows<T, HPW, 16>(a, T_rows, blocks_z, warps, smem, st);
}

}  // namespace gi

using namespace gi;

extern "C" int gi_attention_rows_supported(int hd, int vd) {
    return hd >= 1 && hd <= kRowsMaxHeadDim && vd >= 1 && vd <= kRowsMaxValueDim;
}

static int gi_attention_rows_impl(const void* q, int q_dtype, int ldq, const void* k_cache, const void* v_cache, int cache_dtype,
                                 void* out, int out_dtype, int ldo, const int* row_req, const int* positions,
                                 const int* block_tables, int table_stride, int T, int H, int Hkv, int hd, int vd, int v_row,
                                 int values_in_keys, int page_size, float scale, int window, int chunk, const float* slopes,
                                 const float* sinks, void* stream) {
    if (T == 0) return 0;
    GI_REQUIRE(T > 0 && H > 0 && Hkv > 0 && page_size > 0, "attention_rows: sizes must be positive");
    GI_REQUIRE(H % Hkv == 0, "attention_rows: %d query heads are not a multiple of %d key/value heads", H, Hkv);
    GI_REQUIRE(gi_attention_rows_supported(hd, vd), "attention_rows: head size %d / value size %d is not supported (up to %d / %d)",
               hd, vd, kRowsMaxHeadDim, kRowsMaxValueDim);
    GI_REQUIRE(!values_in_keys || (vd <= hd && v_row == hd), "attention_rows: values inside the key rows must fit them");
    GI_REQUIRE(v_row >= vd && ldq >= H * hd && ldo >= H * vd, "attention_rows: a row is shorter than its heads");
    GI_REQUIRE(Hkv <= 65535, "attention_rows: too many key/value heads for one launch");
    GI_REQUIRE((q_dtype == kF32 || q_dtype == kBF16) && (out_dtype == kF32 || out_dtype == kBF16) &&
               (cache_dtype == kF32 || cache_dtype == kBF16), "attention_rows: unsupported dtype code");
    const int group = H / Hkv;
    RowsArgs a;
    a.q = q; a.q_is_f32 = q_dtype == kF32; a.ldq = ldq;
    a.k_cache = k_cache; a.v_cache = values_in_keys ? k_cache : v_cache;
    a.out = out; a.out_is_f32 = out_dtype == kF32; a.ldo = ldo;
    a.row_req = row_req; a.positions = positions; a.block_tables = block_tables; a.table_stride = table_stride;
    a.H = H; a.Hkv = Hkv; a.hd = hd; a.vd = vd; a.v_row = v_row; a.page_size = page_size;
    a.scale = scale; a.window = window; a.chunk = chunk; a.slopes = slopes; a.sinks = sinks;
    a.alias = values_in_keys ? 1 : 0;
    // rows of the key tile: pairs of values are read by 32 lanes from 32 rows, free of bank conflicts when the row
    // length counted in pairs is odd
    const int hdp = (hd + 1) & ~1;
    a.ks = (hdp / 2) % 2 ? hdp : hdp + 2;
    // few heads in a group: a warp per head; many: four heads per warp, up to sixteen per block
    const int hpw = group <= 4 ? 1 : 4;
    a.heads_per_block = group <= 4 ? group : std::min((group + 3) / 4 * 4, 16);
    const int warps = a.heads_per_block / hpw;
    const int blocks_z = (group + a.heads_per_block - 1) / a.heads_per_block;
    const size_t esz = cache_dtype == kF32 ? 4 : 2;
    const size_t smem = static_cast<size_t>(a.heads_per_block) * hdp * 4 + static_cast<size_t>(kRowsTile) * a.ks * esz +
                        (a.alias ? 0 : static_cast<size_t>(kRowsTile) * vd * esz);
    GI_REQUIRE(smem <= 200 * 1024, "attention_rows: head size %d with %d heads per block needs %zu bytes of shared memory", hd,
               a.heads_per_block, smem);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int rows_left = T;
    GI_REQUIRE(rows_left <= 2147483647, "attention_rows: too many rows");
    if (cache_dtype == kF32)
        return hpw == 1 ? launch_rows_vi<float, 1>(a, T, blocks_z, warps, smem, st) : launch_rows_vi<float, 4>(a, T, blocks_z, warps, smem, st);
    return hpw == 1 ? launch_rows_vi<__nv_bfloat16, 1>(a, T, blocks_z, warps, smem, st)
                    : launch_rows_vi<__nv_bfloat16, 4>(a, T, blocks_z, warps, smem, st);
}

extern "C" int gi_attention_rows(const void* q, int q_dtype, int ldq, const void* k_cache, const void* v_cache, int cache_dtype,
                                 void* out, int out_dtype, int ldo, const int* row_req, const int* positions,
                                 const int* block_tables, int table_stride, int T, int H, int Hkv, int hd, int vd, int v_row,
                                 int values_in_keys, int page_size, float scale, int window, int chunk, const float* slopes,
                                 const float* sinks, void* stream) {
    return gi::dispatch(gi_attention_rows_impl, q, q_dtype, ldq, k_cache, v_cache, cache_dtype, out, out_dtype, ldo, row_req,
                        positions, block_tables, table_stride, T, H, Hkv, hd, vd, v_row, values_in_keys, page_size, scale, window,
                        chunk, slopes, sinks, stream);
}
