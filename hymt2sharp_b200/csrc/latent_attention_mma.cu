// bfloat16 attention over a cache of ONE vector per token that all heads share (see hymt2_attention_shared_vector:
// every head's key is the whole row of width d, every head's value its first dv entries), on the tensor cores through
// warp-level matrix fragments (16x16x16, float32 accumulation).  Prompts, portions of prompts and decode steps.
//
// Because all heads read the same keys, the (token, head) pairs of a sequence are simply the consecutive rows of
// q [T * heads, d]: a block owns 64 of them and walks the keys in tiles of 64, which is one cache block and therefore
// one contiguous piece of memory.  Per tile: S = Q K^T into shared memory; the online softmax on S in float32 (the
// row's running maximum and sum, the factor that the old sums shrink by); P in bfloat16; O = O * factor + P V with
// O [64, dv] held in accumulator fragments.  How the entries of an accumulator fragment map to rows is found out once,
// by loading a matrix whose entries are their own row numbers.
// Row r of sequence b (token r / heads of its new tokens) sits at position p = kv_len - n_b + r / heads and sees the
// keys max(0, p - window + 1) .. p.  With split_keys > 0 (decode steps) a block takes one chunk of that many keys
// and leaves unnormalised partials, which the merge kernel of the CUDA-core attention folds in chunk order.
//
// The same kernel has a second form (EXPANDED) for prompts that start at position 0, where every key of a sequence is
// one of the step's own tokens: keys and values are then worth rebuilding per head (K_h = [W_uk[h] c | rotated part],
// V_h = W_uv[h] c, made by one product for all tokens) because a head's rows are several times narrower than the
// compressed row.  A block then owns 64 TOKENS of ONE head; queries, keys and values are read from the matrices that
// the projections left, the key tile is put together from the head's own columns and the shared rotated part, and the
// values have a tile of their own.
#include "common.cuh"

#include <mma.h>

int hymt2_attention_merge_launch(void* out, int dtype, const int* cu_seqlens, const int* slot_ids, const int* kv_lens,
                                 float* part_acc, float* part_ml, int tokens, int nh, int d, int window, int split_keys,
                                 int max_splits, cudaStream_t stream, int* status);

namespace {

using namespace nvcuda;
typedef __nv_bfloat16 bf16;

constexpr int MT = 64, NT = 64, THREADS = 256, S_LD = 68, P_LD = 72;

// 16 bytes from global to shared memory without a stop in registers; `valid` false: 16 zero bytes (nothing is read, the
// address only has to be one that exists).  A tile's copies are all issued before any is waited for.
__device__ __forceinline__ void copy16_async(void* smem, const void* gmem, bool valid) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void copies_wait() { asm volatile("cp.async.wait_all;" ::: "memory"); }

struct LatentMmaParams {
    const bf16* q;        // [T * nh, d]
    bf16* out;            // [T * nh, dv]
    const bf16* cache;    // plane base, [block][64][d]
    const int* block_table;
    const int* cu_seqlens;
    const int* slot_ids;
    const int* kv_lens;
    float* part_acc;      // [T * nh, splits, dv]
    float* part_ml;       // [T * nh, splits, 2]
    int table_stride, nh, d, dv, window, split_keys, max_splits;
    float scale;
    // the expanded form: q is the projection [T, ldq_g] with head h's d entries at column h * d; out is [T, ld_out]
    const bf16* kexp;     // [T, ld_kexp]: head h's unrotated key entries at column h * dim
    const bf16* vexp;     // [T, ld_vexp]: head h's values at column h * dv
    const bf16* krot;     // [T, ld_krot]: the rotated key part that all heads share
    long ldq_g, ld_out, ld_kexp, ld_vexp, ld_krot;
    int dim;              // unrotated entries of a key (d - dim are the rotated ones)
};

template <int MAXF, bool EXPANDED>
__global__ void __launch_bounds__(THREADS, EXPANDED ? 2 : 1)
latent_attention_mma_kernel(LatentMmaParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int d = p.d, dv = p.dv, ldq = d + 8;
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);           // [64][ldq]
    bf16* Ks = Qs + MT * ldq;                               // [64][ldq]
    float* Ss = reinterpret_cast<float*>(Ks + NT * ldq);    // [64][S_LD]
    bf16* Ps = reinterpret_cast<bf16*>(Ss + MT * S_LD);     // [64][P_LD]
    float* m_s = reinterpret_cast<float*>(Ps + MT * P_LD);  // [64] running maximum
    float* l_s = m_s + MT;                                  // [64] running sum
    float* corr_s = l_s + MT;                               // [64] what the old sums shrink by in this tile
    bf16* Vs = reinterpret_cast<bf16*>(corr_s + MT);        // [64][dv + 8], the expanded form only
    const int ldv = EXPANDED ? dv + 8 : ldq;
    const int head = EXPANDED ? blockIdx.y : 0;

    const int b = blockIdx.z / p.max_splits, split = blockIdx.z % p.max_splits;
    const int slot = p.slot_ids[b];
    if (slot < 0) return;
    const int tok0 = p.cu_seqlens[b], n = p.cu_seqlens[b + 1] - tok0;
    const int kv_len = p.kv_lens[b], start = kv_len - n;
    // (the tiles with the most keys first: a sequence's last rows see all of it)
    const int rows_total = EXPANDED ? n : n * p.nh, r0 = (int)(gridDim.x - 1 - blockIdx.x) * MT;
    if (r0 >= rows_total) return;
    const int rows_valid = min(MT, rows_total - r0);
    const int first_tok = EXPANDED ? r0 : r0 / p.nh, last_tok = EXPANDED ? r0 + rows_valid - 1 : (r0 + rows_valid - 1) / p.nh;
    int key_end = start + last_tok + 1;
    int key_begin = p.window > 0 ? max(0, start + first_tok - p.window + 1) : 0;
    if (p.split_keys > 0) {
        key_begin = max(key_begin, split * p.split_keys);
        key_end = min(key_end, (split + 1) * p.split_keys);
    }
    if (key_begin >= key_end) return;   // (no row of this tile sees a key of this chunk; the merge never asks for it)

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const size_t row_base = (size_t)tok0 * p.nh + r0;     // first of this tile's rows among all (token, head) rows

    // the queries
    const bf16* qg = EXPANDED ? p.q + (size_t)(tok0 + r0) * p.ldq_g + (size_t)head * d : p.q + row_base * d;
    const size_t q_ld = EXPANDED ? (size_t)p.ldq_g : (size_t)d;
    // A thread's 16-byte pieces of a [rows][d] tile are THREADS * 8 entries apart: row and column move on by fixed
    // steps (one division for the kernel, none per piece).
    const int step_r = (THREADS * 8) / d, step_c = (THREADS * 8) - step_r * d;
    const int first_r = (tid * 8) / d, first_c = tid * 8 - first_r * d;
    const int q_rows = min(MT, (rows_valid + 15) & ~15);   // whole row fragments that hold a live row; the others are never read
    for (int r = first_r, c = first_c; r < q_rows;) {
        const bool ok = r < rows_valid;
        copy16_async(Qs + r * ldq + c, qg + (ok ? (size_t)r * q_ld + c : 0), ok);
        r += step_r; c += step_c;
        if (c >= d) { c -= d; r++; }
    }
    if (tid < MT) { m_s[tid] = -INFINITY; l_s[tid] = 0.f; corr_s[tid] = 1.f; }

    // which row of its 16 each entry of an accumulator fragment belongs to
    // A tile of at most 16 live rows (a decode step's heads) is `narrow`: all warps share the one live row fragment and
    // divide the columns among themselves; otherwise a warp owns one of four row fragments and every second column fragment.
    const bool narrow = rows_valid <= 16;
    const int rf_o = narrow ? 0 : warp & 3;                 // this warp's row fragment of O,
    const int cf_o = narrow ? warp : warp >> 2;             // its first column fragment
    const int cf_step = narrow ? 8 : 2;                     // and the distance to its next
    const int o_col_frags = dv >> 4;
    float* stage = Ss + (warp & 3) * 16 * S_LD + (warp >> 2) * 16;   // a 16x16 float32 patch of S that only this warp touches outside the S phase
    int row_of[8];
    {
        for (int i = lane; i < 256; i += 32) stage[(i >> 4) * S_LD + (i & 15)] = (float)(i >> 4);
        __syncwarp();
        wmma::fragment<wmma::accumulator, 16, 16, 16, float> probe;
        wmma::load_matrix_sync(probe, stage, S_LD, wmma::mem_row_major);
#pragma unroll
        for (int e = 0; e < 8; e++) row_of[e] = (int)probe.x[e];
    }
    wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc[MAXF];   // O: row fragment rf_o, column fragments cf_o + i * cf_step
#pragma unroll
    for (int i = 0; i < MAXF; i++) wmma::fill_fragment(acc[i], 0.f);
    const bool o_rows_live = rf_o * 16 < rows_valid;
    // this warp's part of S: row fragment rf_s, column fragments cf_s, cf_s + 1 (narrow: warps 0..3 take one column fragment each)
    // In the narrow layout warps 0..3 sum over the first half of a key's entries and warps 4..7 over the second half, into rows
    // 16..31 of S; the softmax adds the two.
    const int rf_s = narrow ? 0 : warp >> 1, cf_s = narrow ? (warp & 3) : (warp & 1) * 2;
    const bool s_rows_live = narrow ? true : rf_s * 16 < rows_valid;
    const int kk_half = ((d >> 4) + 1) >> 1 << 4;   // entries that the first half takes (whole pieces of 16)
    const int kk_begin = narrow && warp >= 4 ? kk_half : 0, kk_end = narrow && warp < 4 ? kk_half : d;
    const int s_row0 = narrow && warp >= 4 ? 16 : rf_s * 16;

    const int* table = p.block_table + (size_t)slot * p.table_stride;
    for (int k0 = (key_begin / NT) * NT; k0 < key_end; k0 += NT) {
        __syncthreads();   // the tile before is done with Ks and Ps (and, first time round, Qs and the statistics are written)
        if (EXPANDED) {
            const int keys_here = min(NT, n - k0);   // (the sequence starts in this step: its keys are its new tokens)
            const size_t t0 = (size_t)tok0 + k0;
            for (int r = first_r, c = first_c; r < NT;) {
                const bool ok = r < keys_here;
                const size_t t = t0 + (ok ? r : 0);
                copy16_async(Ks + r * ldq + c, c < p.dim ? p.kexp + t * p.ld_kexp + (size_t)head * p.dim + c : p.krot + t * p.ld_krot + (c - p.dim), ok);
                r += step_r; c += step_c;
                if (c >= d) { c -= d; r++; }
            }
            for (int i = tid * 8; i < NT * dv; i += THREADS * 8) {
                const int r = i / dv, c = i - r * dv;
                const bool ok = r < keys_here;
                copy16_async(Vs + r * ldv + c, p.vexp + (t0 + (ok ? r : 0)) * p.ld_vexp + (size_t)head * dv + c, ok);
            }
        } else {
            const int block = table[k0 / NT];
            const bf16* kg = p.cache + (size_t)(block < 0 ? 0 : block) * NT * d;
            const int keys_here = block < 0 ? 0 : min(NT, kv_len - k0);   // rows past the sequence's end hold anything: they are zeroed
            for (int r = first_r, c = first_c; r < NT;) {
                const bool ok = r < keys_here;
                copy16_async(Ks + r * ldq + c, kg + (ok ? (size_t)r * d + c : 0), ok);
                r += step_r; c += step_c;
                if (c >= d) { c -= d; r++; }
            }
        }
        copies_wait();
        __syncthreads();

        // S = Q K^T
        if (s_rows_live) {
            wmma::fragment<wmma::accumulator, 16, 16, 16, float> s0, s1;
            wmma::fill_fragment(s0, 0.f);
            wmma::fill_fragment(s1, 0.f);
            const bf16* qa = Qs + rf_s * 16 * ldq;
            const bf16* kb0 = Ks + cf_s * 16 * ldq;
            const bf16* kb1 = kb0 + 16 * ldq;
            for (int kk = kk_begin; kk < kk_end; kk += 16) {
                wmma::fragment<wmma::matrix_a, 16, 16, 16, bf16, wmma::row_major> a;
                wmma::fragment<wmma::matrix_b, 16, 16, 16, bf16, wmma::col_major> b0, b1;
                wmma::load_matrix_sync(a, qa + kk, ldq);
                wmma::load_matrix_sync(b0, kb0 + kk, ldq);
                wmma::mma_sync(s0, a, b0, s0);
                if (!narrow) {
                    wmma::load_matrix_sync(b1, kb1 + kk, ldq);
                    wmma::mma_sync(s1, a, b1, s1);
                }
            }
            wmma::store_matrix_sync(Ss + s_row0 * S_LD + cf_s * 16, s0, S_LD, wmma::mem_row_major);
            if (!narrow) wmma::store_matrix_sync(Ss + s_row0 * S_LD + cf_s * 16 + 16, s1, S_LD, wmma::mem_row_major);
        }
        __syncthreads();

        // the online softmax: four threads a row, 16 keys each (narrow: the 16 live rows only)
        if (!narrow || tid < 64) {
            const int r = tid >> 2, part = tid & 3;
            const int grow = r0 + r;
            const bool row_ok = r < rows_valid;
            const int pos = start + (EXPANDED ? grow : grow / p.nh);
            const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
            float s[16];
            float tmax = -INFINITY;
#pragma unroll
            for (int j = 0; j < 16; j++) {
                const int key = k0 + part * 16 + j;
                const bool visible = row_ok && key >= lo && key <= pos && key >= key_begin && key < key_end;
                const float sum = narrow ? Ss[r * S_LD + part * 16 + j] + Ss[(16 + r) * S_LD + part * 16 + j] : Ss[r * S_LD + part * 16 + j];
                s[j] = visible ? sum * p.scale : -INFINITY;
                tmax = fmaxf(tmax, s[j]);
            }
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
            const float m_old = m_s[r], m_new = fmaxf(m_old, tmax);
            float corr = 1.f, psum = 0.f;
            __nv_bfloat162 pb[8];
            if (m_new > -INFINITY) {
                corr = expf(m_old - m_new);
#pragma unroll
                for (int j = 0; j < 16; j += 2) {
                    const float p0 = expf(s[j] - m_new), p1 = expf(s[j + 1] - m_new);
                    psum += p0 + p1;
                    pb[j >> 1] = __floats2bfloat162_rn(p0, p1);
                }
            } else {
#pragma unroll
                for (int j = 0; j < 8; j++) pb[j] = __floats2bfloat162_rn(0.f, 0.f);
            }
            psum += __shfl_xor_sync(0xffffffffu, psum, 1);
            psum += __shfl_xor_sync(0xffffffffu, psum, 2);
            uint4* dst = reinterpret_cast<uint4*>(Ps + r * P_LD + part * 16);
            dst[0] = *reinterpret_cast<uint4*>(&pb[0]);
            dst[1] = *reinterpret_cast<uint4*>(&pb[4]);
            __syncwarp();
            if (part == 0) {
                m_s[r] = m_new;
                l_s[r] = l_s[r] * corr + psum;
                corr_s[r] = corr;
            }
        }
        __syncthreads();

        // O = O * factor + P V (the values are the first dv entries of the key rows)
        if (o_rows_live) {
            float f[8];
#pragma unroll
            for (int e = 0; e < 8; e++) f[e] = corr_s[rf_o * 16 + row_of[e]];
#pragma unroll
            for (int i = 0; i < MAXF; i++)
                if (cf_o + cf_step * i < o_col_frags) {
#pragma unroll
                    for (int e = 0; e < 8; e++) acc[i].x[e] *= f[e];
                }
#pragma unroll
            for (int kk = 0; kk < NT; kk += 16) {
                wmma::fragment<wmma::matrix_a, 16, 16, 16, bf16, wmma::row_major> a;
                wmma::load_matrix_sync(a, Ps + rf_o * 16 * P_LD + kk, P_LD);
#pragma unroll
                for (int i = 0; i < MAXF; i++)
                    if (cf_o + cf_step * i < o_col_frags) {
                        wmma::fragment<wmma::matrix_b, 16, 16, 16, bf16, wmma::row_major> vb;
                        wmma::load_matrix_sync(vb, (EXPANDED ? Vs : Ks) + kk * ldv + (cf_o + cf_step * i) * 16, ldv);
                        wmma::mma_sync(acc[i], a, vb, acc[i]);
                    }
            }
        }
    }
    __syncthreads();

    const bool split_mode = p.split_keys > 0;
    if (split_mode && tid < rows_valid) {
        float* ml = p.part_ml + ((row_base + tid) * p.max_splits + split) * 2;
        ml[0] = m_s[tid];
        ml[1] = l_s[tid];
    }
    if (!o_rows_live) return;
    float f[8];
#pragma unroll
    for (int e = 0; e < 8; e++) {
        const float l = l_s[rf_o * 16 + row_of[e]];
        f[e] = split_mode ? 1.f : (l > 0.f ? 1.0f / l : 0.f);
    }
#pragma unroll
    for (int i = 0; i < MAXF; i++) {
        if (cf_o + cf_step * i >= o_col_frags) continue;
#pragma unroll
        for (int e = 0; e < 8; e++) acc[i].x[e] *= f[e];
        wmma::store_matrix_sync(stage, acc[i], S_LD, wmma::mem_row_major);
        __syncwarp();
        const int r = lane >> 1, c8 = (lane & 1) * 8;
        const int row = rf_o * 16 + r, col = (cf_o + cf_step * i) * 16 + c8;
        if (row < rows_valid) {
            const float* src = stage + r * S_LD + c8;
            if (split_mode) {
                float* dst = p.part_acc + ((row_base + row) * p.max_splits + split) * dv + col;
#pragma unroll
                for (int e = 0; e < 8; e++) dst[e] = src[e];
            } else {
                __nv_bfloat162 h[4];
#pragma unroll
                for (int e = 0; e < 4; e++) h[e] = __floats2bfloat162_rn(src[2 * e], src[2 * e + 1]);
                bf16* dst = EXPANDED ? p.out + (size_t)(tok0 + r0 + row) * p.ld_out + (size_t)head * dv + col : p.out + (row_base + row) * dv + col;
                *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<uint4*>(h);
            }
        }
        __syncwarp();
    }
}

size_t smem_bytes(int d, int dv_tile = 0) {
    return (size_t)2 * MT * (d + 8) * sizeof(bf16) + (size_t)MT * S_LD * sizeof(float) + (size_t)MT * P_LD * sizeof(bf16) + 3 * MT * sizeof(float)
         + (dv_tile ? (size_t)NT * (dv_tile + 8) * sizeof(bf16) : 0);
}

}  // namespace

// Whether the kernel takes these sizes: rows of 16-element pieces, cache blocks of 64 tokens, and room in shared memory.
HYMT2_API int hymt2_latent_attention_mma_supported(int d, int dv, int block_tokens) {
    return d > 0 && dv > 0 && d % 16 == 0 && dv % 16 == 0 && dv <= d && dv <= 512 && block_tokens == NT && smem_bytes(d) <= 220 * 1024;
}

HYMT2_API int hymt2_latent_attention_mma(void* out, const void* q, const void* cache, const int* block_table, int table_stride,
                                         int block_tokens, const int* cu_seqlens, const int* slot_ids, const int* kv_lens, int batch,
                                         int tokens, int max_new_tokens, int nh, int d, int dv, float scale, int window,
                                         int split_keys, int max_splits, float* part_acc, float* part_ml, int* status,
                                         cudaStream_t stream) {
    if (batch == 0 || tokens == 0) return HYMT2_OK;
    HYMT2_REQUIRE(hymt2_latent_attention_mma_supported(d, dv, block_tokens), "latent_attention_mma: keys of %d, values of %d, blocks of %d are not taken", d, dv, block_tokens);
    HYMT2_REQUIRE(batch > 0 && tokens > 0 && nh > 0 && max_new_tokens > 0, "latent_attention_mma: bad sizes");
    HYMT2_REQUIRE((uintptr_t)q % 16 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)cache % 16 == 0, "latent_attention_mma: operands must be 16-byte aligned");
    HYMT2_REQUIRE(split_keys == 0 || (split_keys % NT == 0 && max_splits > 0 && part_acc && part_ml), "latent_attention_mma: a split comes in whole tiles and with scratch");
    LatentMmaParams p;
    p.q = (const bf16*)q; p.out = (bf16*)out; p.cache = (const bf16*)cache; p.block_table = block_table; p.cu_seqlens = cu_seqlens;
    p.slot_ids = slot_ids; p.kv_lens = kv_lens; p.part_acc = part_acc; p.part_ml = part_ml; p.table_stride = table_stride; p.nh = nh;
    p.d = d; p.dv = dv; p.window = window; p.split_keys = split_keys; p.max_splits = split_keys > 0 ? max_splits : 1; p.scale = scale;
    const long row_tiles = ((long)max_new_tokens * nh + MT - 1) / MT;
    HYMT2_REQUIRE(row_tiles <= 2147483647L && (long)batch * p.max_splits <= 65535, "latent_attention_mma: grid too large");
    const dim3 grid((unsigned)row_tiles, 1, (unsigned)(batch * p.max_splits));
    const size_t smem = smem_bytes(d);
    auto launch = [&](auto kernel) -> int {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) { hymt2_set_error("latent_attention_mma: %s", cudaGetErrorString(e)); return HYMT2_ERR_LAUNCH; }
        kernel<<<grid, THREADS, smem, stream>>>(p);
        return hymt2_check_launch("latent_attention_mma");
    };
    int rc;
    if (dv <= 128) rc = launch(latent_attention_mma_kernel<4, false>);
    else if (dv <= 256) rc = launch(latent_attention_mma_kernel<8, false>);
    else rc = launch(latent_attention_mma_kernel<16, false>);
    if (rc == HYMT2_OK && split_keys > 0)
        rc = hymt2_attention_merge_launch(out, HYMT2_BF16, cu_seqlens, slot_ids, kv_lens, part_acc, part_ml, tokens, nh, dv, window,
                                          split_keys, max_splits, stream, status);
    return rc;
}

// The expanded form (see the head of this file): whole prompts from position 0 with per-head keys and values.
HYMT2_API int hymt2_latent_attention_expanded_supported(int dim, int rot, int dv) {
    const int d = dim + rot;
    return dim > 0 && rot >= 0 && dv > 0 && d % 16 == 0 && dv % 16 == 0 && dim % 8 == 0 && dv <= 256 && smem_bytes(d, dv) <= 110 * 1024;
}

HYMT2_API int hymt2_latent_attention_expanded(void* out, long ld_out, const void* q, long ldq, const void* kexp, long ld_kexp,
                                              const void* vexp, long ld_vexp, const void* krot, long ld_krot,
                                              const int* cu_seqlens, const int* slot_ids, const int* kv_lens, int batch,
                                              int max_new_tokens, int nh, int dim, int rot, int dv, float scale, int window,
                                              cudaStream_t stream) {
    if (batch == 0 || max_new_tokens == 0) return HYMT2_OK;
    HYMT2_REQUIRE(hymt2_latent_attention_expanded_supported(dim, rot, dv), "latent_attention_expanded: heads of %d + %d key entries and %d value entries are not taken", dim, rot, dv);
    HYMT2_REQUIRE(batch > 0 && batch <= 65535 && nh > 0 && nh <= 65535, "latent_attention_expanded: bad sizes");
    const uintptr_t bits = (uintptr_t)out | (uintptr_t)q | (uintptr_t)kexp | (uintptr_t)vexp | (uintptr_t)krot;
    HYMT2_REQUIRE(bits % 16 == 0 && ld_out % 8 == 0 && ldq % 8 == 0 && ld_kexp % 8 == 0 && ld_vexp % 8 == 0 && ld_krot % 8 == 0,
                  "latent_attention_expanded: operands and rows must be 16-byte aligned");
    LatentMmaParams p = {};
    p.q = (const bf16*)q; p.out = (bf16*)out; p.cu_seqlens = cu_seqlens; p.slot_ids = slot_ids; p.kv_lens = kv_lens;
    p.nh = nh; p.d = dim + rot; p.dv = dv; p.window = window; p.split_keys = 0; p.max_splits = 1; p.scale = scale;
    p.kexp = (const bf16*)kexp; p.vexp = (const bf16*)vexp; p.krot = (const bf16*)krot;
    p.ldq_g = ldq; p.ld_out = ld_out; p.ld_kexp = ld_kexp; p.ld_vexp = ld_vexp; p.ld_krot = ld_krot; p.dim = dim;
    const dim3 grid((max_new_tokens + MT - 1) / MT, nh, batch);
    const size_t smem = smem_bytes(p.d, dv);
    auto launch = [&](auto kernel) -> int {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) { hymt2_set_error("latent_attention_expanded: %s", cudaGetErrorString(e)); return HYMT2_ERR_LAUNCH; }
        kernel<<<grid, THREADS, smem, stream>>>(p);
        return hymt2_check_launch("latent_attention_expanded");
    };
    return dv <= 128 ? launch(latent_attention_mma_kernel<4, true>) : launch(latent_attention_mma_kernel<8, true>);
}
