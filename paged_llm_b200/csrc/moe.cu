// A feed-forward of routed experts: router, the list of (token, expert) pairs sorted by expert, the
// experts' products over that list, and the weighted sum.
//
//   z = W_r h (float32, a product of the kernel library);  the k largest z choose the experts;  their weights
//   are the softmax over those k;
//   y = sum_j weight_j * down_e(j)(act(gate_e(j) h) * up_e(j) h)  [+ sigmoid(w_s . h) * shared(h)]
//
// Nothing here looks at the batch on the host: the counts per expert stay on the device, every kernel is
// launched for the most tiles the step can have and blocks beyond the real count leave at once, so a step
// can be captured and replayed.  A pair is (token t, choice j), numbered t * k + j; tiles of BM pairs of one
// expert are listed in `sorted` (padded per expert with -1) and `tile_expert`.
#include <cuda_bf16.h>

#include "common.cuh"

namespace {

// act(gate) * up; activation 2 is the clamped one (common.cuh: gated_act_f).
__device__ __forceinline__ float act_mul_f(int act, float limit, float g, float u) { return gated_act_f(act, limit, g, u); }

// ------------------------------------------------------------------ the router's choice
// The logits z[t][0..E) (and, if `shared_gate`, z[t][E], whose sigmoid is the token's factor for the shared
// expert) come from a product of the kernel library in float32.  One warp per token picks the k largest, one
// after the other (among equals the lowest index), and forms the softmax over the chosen.
__global__ void __launch_bounds__(128) moe_topk_kernel(const float* __restrict__ z_all, int ldz, int tokens, int E, int k,
                                                       int shared_gate, int* __restrict__ top_idx,
                                                       float* __restrict__ top_w, float* __restrict__ gate) {
    extern __shared__ float z_smem[];                   // [4][E]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + warp;
    if (t >= tokens) return;
    float* z = z_smem + warp * E;
    const float* src = z_all + (size_t)t * ldz;
    for (int e = lane; e < E; e += 32) z[e] = src[e];
    if (shared_gate && lane == 0) gate[t] = 1.0f / (1.0f + expf(-src[E]));
    __syncwarp();
    float chosen_z = 0.f, z_max = 0.f;
    int chosen_e = -1;                                  // lane j keeps choice j (k <= 32)
    for (int j = 0; j < k; ++j) {
        float best = -INFINITY;
        int arg = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = z[e];
            if (v > best || (v == best && e < arg)) {
                best = v;
                arg = e;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) {
                best = ob;
                arg = oa;
            }
        }
        if (arg >= E) arg = 0;                          // (only if every logit left is NaN)
        if (j == 0) z_max = best;
        if (lane == j) {
            chosen_z = best;
            chosen_e = arg;
        }
        __syncwarp();
        if (lane == 0) z[arg] = -INFINITY;
        __syncwarp();
    }
    const float pj = lane < k ? expf(chosen_z - z_max) : 0.f;
    const float sum = warp_sum(pj);
    if (lane < k) {
        top_idx[(size_t)t * k + lane] = chosen_e;
        top_w[(size_t)t * k + lane] = pj / sum;
    }
}

// The arg-max of v[0..n) over a warp (among equals the lowest index); every lane gets the result.
__device__ __forceinline__ void warp_argmax(const float* v, int n, int lane, float& best, int& arg) {
    best = -INFINITY;
    arg = 0x7fffffff;
    for (int e = lane; e < n; e += 32) {
        const float x = v[e];
        if (x > best || (x == best && e < arg)) {
            best = x;
            arg = e;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
        if (ob > best || (ob == best && oa < arg)) {
            best = ob;
            arg = oa;
        }
    }
    if (arg >= n) arg = 0;                              // (only if every value left is NaN)
}

// Choice by sigmoid scores: s = sigmoid(z) per expert; with groups (count > 0) the experts form `count` equal groups
// of neighbours, a group scores the sum of its `group_top` largest s, and only experts of the `keep` best groups can be
// chosen; the k largest s among those choose the experts, and the weights are those s as they are.  One warp per token.
__global__ void __launch_bounds__(128) moe_sigmoid_topk_kernel(const float* __restrict__ z_all, int ldz, int tokens, int E, int k,
                                                               int count, int keep, int group_top, int* __restrict__ top_idx,
                                                               float* __restrict__ top_w) {
    extern __shared__ float z_smem[];                   // per warp: scores [E], what may still be chosen [E], group scores [E]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + warp;
    if (t >= tokens) return;
    float* sc = z_smem + (size_t)warp * 3 * E;
    float* pick = sc + E;
    float* gsc = pick + E;
    const float* src = z_all + (size_t)t * ldz;
    for (int e = lane; e < E; e += 32) pick[e] = sc[e] = 1.0f / (1.0f + expf(-src[e]));
    __syncwarp();
    if (count > 0) {
        const int size = E / count;
        // a lane per group: the sum of the group's `group_top` largest scores, taken one after the other
        for (int g = lane; g < count; g += 32) {
            float sum = 0.f;
            int taken[8];                               // group_top <= 8
            for (int r = 0; r < group_top && r < size; ++r) {
                float best = -INFINITY;
                int arg = -1;
                for (int i = 0; i < size; ++i) {
                    bool used = false;
                    for (int q = 0; q < r; ++q) used |= taken[q] == i;
                    const float x = sc[g * size + i];
                    if (!used && x > best) {
                        best = x;
                        arg = i;
                    }
                }
                taken[r] = arg;
                sum += best;
            }
            gsc[g] = sum;
        }
        __syncwarp();
        // the best groups stay; their score is taken out as they are found, the others' experts cannot be chosen
        for (int r = 0; r < keep; ++r) {
            float best;
            int arg;
            warp_argmax(gsc, count, lane, best, arg);
            __syncwarp();
            if (lane == 0) gsc[arg] = -INFINITY;
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (gsc[e / size] != -INFINITY) pick[e] = -1.0f;
        __syncwarp();
    }
    for (int j = 0; j < k; ++j) {
        float best;
        int arg;
        warp_argmax(pick, E, lane, best, arg);
        __syncwarp();
        if (lane == 0) {
            top_idx[(size_t)t * k + j] = arg;
            top_w[(size_t)t * k + j] = sc[arg];
            pick[arg] = -INFINITY;
        }
        __syncwarp();
    }
}

// ------------------------------------------------------------------ pairs sorted by expert
// One block.  sorted[cap]: the pairs of expert 0, padded with -1 to a multiple of BM, then those of expert
// 1, ...; tile_expert[i]: the expert of tile i; *n_tiles: the tiles in use; place[i] (may be null): where pair
// i stands in `sorted`.
__global__ void __launch_bounds__(1024) moe_align_kernel(const int* __restrict__ top_idx, int n_pairs, int E, int BM,
                                                         int cap, int* __restrict__ sorted, int* __restrict__ tile_expert,
                                                         int* __restrict__ n_tiles, int* __restrict__ place) {
    __shared__ int cnt[1024], off[1025];
    const int tid = threadIdx.x;
    for (int e = tid; e < E; e += blockDim.x) cnt[e] = 0;
    for (int i = tid; i < cap; i += blockDim.x) sorted[i] = -1;
    __syncthreads();
    for (int i = tid; i < n_pairs; i += blockDim.x) {
        const int e = top_idx[i];
        if (e >= 0 && e < E) atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    if (tid == 0) {
        int run = 0;
        for (int e = 0; e < E; ++e) {
            off[e] = run;
            run += (cnt[e] + BM - 1) / BM * BM;
        }
        off[E] = run;
        *n_tiles = run / BM;
    }
    __syncthreads();
    for (int e = tid; e < E; e += blockDim.x) {
        for (int i = off[e] / BM; i < off[e + 1] / BM; ++i) tile_expert[i] = e;
        cnt[e] = 0;
    }
    __syncthreads();
    for (int i = tid; i < n_pairs; i += blockDim.x) {
        const int e = top_idx[i];
        if (e >= 0 && e < E) {
            const int at = off[e] + atomicAdd(&cnt[e], 1);
            if (at < cap) sorted[at] = i;
            if (place != nullptr) place[i] = at < cap ? at : -1;
        } else if (place != nullptr) {
            place[i] = -1;
        }
    }
}

// ------------------------------------------------------------------ the experts' products
struct MoeGemm {
    const void* A;              // rows of the left operand; pair i reads row i / a_div
    const void* W;              // [E][rows_w][K]: rows_w = 2 N (gate rows, then up rows) if gated, else N
    void* out;                  // gated: [pairs][ldo] in the compute type; else float32 [pairs][ldo]
    const int* sorted;
    const int* tile_expert;
    const int* n_tiles;
    const float* row_scale;     // [pairs] or null: the result of pair i is multiplied by it
    int lda, a_div, ldo, n_pairs, N, K, act;
    float act_limit;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

constexpr int MG_BN = 64, MG_BK = 64, MG_PITCH = MG_BK + 8, MG_STAGES = 3;

template <int BM, bool GATED>
constexpr int moe_gemm_smem() { return MG_STAGES * (BM + (GATED ? 2 : 1) * MG_BN) * MG_PITCH * 2; }

// bfloat16 on the tensor cores (mma.sync m16n8k16, float32 accumulation).  grid: (tiles, ceil(N / 64)); a
// block takes BM pairs of one expert and 64 columns (gated: 64 gate and the 64 matching up columns);
// operands come in through a ring of three cp.async stages of 64 k each, zero-filled outside the matrices.
// BM = 64: four warps of 16 rows; BM = 16 (few pairs per expert: decoding): four warps of 16 columns.
template <int BM, bool GATED>
__global__ void __launch_bounds__(128) moe_gemm_bf16_kernel(MoeGemm p) {
    constexpr int BN = MG_BN, BK = MG_BK, PITCH = MG_PITCH, STAGES = MG_STAGES;
    constexpr int NB = GATED ? 2 : 1;
    constexpr int WM = BM / 16, WNW = 4 / WM, WN = BN / WNW, NF = WN / 8;
    const int tile = blockIdx.x;
    if (tile >= *p.n_tiles) return;
    const int e = p.tile_expert[tile], n0 = blockIdx.y * BN;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* As = reinterpret_cast<__nv_bfloat16*>(smem_raw);           // [STAGES][BM][PITCH]
    __nv_bfloat16* Bs = As + STAGES * BM * PITCH;                             // [STAGES][NB * BN][PITCH]
    __shared__ int rows[BM];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid < BM) {
        const int id = p.sorted[(size_t)tile * BM + tid];
        rows[tid] = id >= 0 && id < p.n_pairs ? id : -1;
    }
    __syncthreads();
    const __nv_bfloat16* A = (const __nv_bfloat16*)p.A;
    const __nv_bfloat16* W = (const __nv_bfloat16*)p.W + (size_t)e * NB * p.N * p.K;
    constexpr int CH = BK / 8;
    auto load_stage = [&](int stage, int k0) {
        __nv_bfloat16* as = As + stage * BM * PITCH;
        __nv_bfloat16* bs = Bs + stage * NB * BN * PITCH;
        for (int i = tid; i < BM * CH; i += 128) {
            const int r = i / CH, c = i - r * CH, kk = k0 + c * 8;
            const bool ok = rows[r] >= 0 && kk < p.K;
            const __nv_bfloat16* src = ok ? A + (size_t)(rows[r] / p.a_div) * p.lda + kk : A;
            cp_async16(as + r * PITCH + c * 8, src, ok ? 16 : 0);
        }
        for (int i = tid; i < NB * BN * CH; i += 128) {
            const int r = i / CH, c = i - r * CH, kk = k0 + c * 8;
            const int which = r / BN, n = n0 + r % BN;
            const bool ok = n < p.N && kk < p.K;
            const __nv_bfloat16* src = ok ? W + ((size_t)which * p.N + n) * p.K + kk : W;
            cp_async16(bs + r * PITCH + c * 8, src, ok ? 16 : 0);
        }
        cp_async_commit();
    };
    float acc[NB][NF][4];
#pragma unroll
    for (int b = 0; b < NB; ++b)
#pragma unroll
        for (int j = 0; j < NF; ++j)
#pragma unroll
            for (int q = 0; q < 4; ++q) acc[b][j][q] = 0.f;
    const int wm = warp % WM, wn = warp / WM;
    const int nk = (p.K + BK - 1) / BK;
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < nk) load_stage(s, s * BK);
        else cp_async_commit();
    }
    for (int kt = 0; kt < nk; ++kt) {
        if (kt + STAGES - 1 < nk) load_stage((kt + STAGES - 1) % STAGES, (kt + STAGES - 1) * BK);
        else cp_async_commit();
        cp_async_wait<STAGES - 1>();
        __syncthreads();
        const __nv_bfloat16* as = As + (kt % STAGES) * BM * PITCH;
        const __nv_bfloat16* bs = Bs + (kt % STAGES) * NB * BN * PITCH;
#pragma unroll
        for (int kk = 0; kk < BK / 16; ++kk) {
            uint32_t a[4];
            ldmatrix_x4(a, as + (wm * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * PITCH + kk * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int b = 0; b < NB; ++b)
#pragma unroll
                for (int n2 = 0; n2 < WN / 16; ++n2) {
                    uint32_t f[4];
                    ldmatrix_x4(f, bs + (b * BN + wn * WN + n2 * 16 + (lane & 7) + (lane >> 4) * 8) * PITCH + kk * 16 +
                                       ((lane >> 3) & 1) * 8);
                    mma_bf16(acc[b][2 * n2], a, f[0], f[1]);
                    mma_bf16(acc[b][2 * n2 + 1], a, f[2], f[3]);
                }
        }
        __syncthreads();
    }
    const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        const int id = rows[wm * 16 + g + 8 * hh];
        if (id < 0) continue;
        const float sc = !GATED && p.row_scale != nullptr ? p.row_scale[id] : 1.f;
#pragma unroll
        for (int j = 0; j < NF; ++j)
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                const int col = n0 + wn * WN + 8 * j + 2 * t4 + q;
                if (col >= p.N) continue;
                if (GATED) {
                    const float v = act_mul_f(p.act, p.act_limit, acc[0][j][2 * hh + q], acc[NB - 1][j][2 * hh + q]);
                    ((__nv_bfloat16*)p.out)[(size_t)id * p.ldo + col] = __float2bfloat16_rn(v);
                } else {
                    ((float*)p.out)[(size_t)id * p.ldo + col] = acc[0][j][2 * hh + q] * sc;
                }
            }
    }
}

// The same on the CUDA cores with one FFMA chain per result in k order, for float32 (true 32-bit) and for
// bfloat16 sizes that the tensor-core form does not take.  Tiles of 16 pairs x 64 columns, 256 threads,
// four columns each.
template <typename T, bool GATED>
__global__ void __launch_bounds__(256) moe_gemm_plain_kernel(MoeGemm p) {
    constexpr int BM = 16, BN = 64, BK = 32, NB = GATED ? 2 : 1;
    const int tile = blockIdx.x;
    if (tile >= *p.n_tiles) return;
    const int e = p.tile_expert[tile], n0 = blockIdx.y * BN;
    __shared__ float As[BM][BK + 1];
    __shared__ float Bs[NB][BK][BN + 1];
    __shared__ int rows[BM];
    const int tid = threadIdx.x;
    if (tid < BM) {
        const int id = p.sorted[(size_t)tile * BM + tid];
        rows[tid] = id >= 0 && id < p.n_pairs ? id : -1;
    }
    __syncthreads();
    const T* A = (const T*)p.A;
    const T* W = (const T*)p.W + (size_t)e * NB * p.N * p.K;
    const int r = tid / 16, c4 = (tid % 16) * 4;
    float acc[NB][4];
#pragma unroll
    for (int b = 0; b < NB; ++b)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[b][j] = 0.f;
    for (int k0 = 0; k0 < p.K; k0 += BK) {
        for (int i = tid; i < BM * BK; i += 256) {
            const int rr = i / BK, kk = i - rr * BK;
            As[rr][kk] = rows[rr] >= 0 && k0 + kk < p.K ? to_float(A[(size_t)(rows[rr] / p.a_div) * p.lda + k0 + kk]) : 0.f;
        }
        for (int i = tid; i < NB * BN * BK; i += 256) {
            const int which = i / (BN * BK), rem = i - which * BN * BK, n = rem / BK, kk = rem - n * BK;
            Bs[which][kk][n] = n0 + n < p.N && k0 + kk < p.K ? to_float(W[((size_t)which * p.N + n0 + n) * p.K + k0 + kk]) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < BK; ++kk) {
            const float a = As[r][kk];
#pragma unroll
            for (int b = 0; b < NB; ++b)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[b][j] = fmaf(a, Bs[b][kk][c4 + j], acc[b][j]);
        }
        __syncthreads();
    }
    const int id = rows[r];
    if (id < 0) return;
    const float sc = !GATED && p.row_scale != nullptr ? p.row_scale[id] : 1.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int col = n0 + c4 + j;
        if (col >= p.N) continue;
        if (GATED) ((T*)p.out)[(size_t)id * p.ldo + col] = from_float<T>(act_mul_f(p.act, p.act_limit, acc[0][j], acc[NB - 1][j]));
        else ((float*)p.out)[(size_t)id * p.ldo + col] = acc[0][j] * sc;
    }
}

// y[t] = sum_j w_j * pair_out[row_j]  (+ gate[t] * shared[t]), float32, with row_j = place[t * k + j] (null:
// t * k + j) and w_j = weight[t * k + j] (null: 1, the rows are weighted already).  pair_out is float32 or (from
// the grouped tensor-core product) bfloat16.
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}

template <typename TP, typename T>
__global__ void moe_combine_kernel(const TP* __restrict__ pair_out, int k, const int* __restrict__ place,
                                   const float* __restrict__ weight, const T* __restrict__ shared,
                                   const float* __restrict__ gate, float* __restrict__ y, int D, int vec) {
    const size_t t = blockIdx.x;
    const float gt = shared != nullptr ? gate[t] : 0.f;
    if (vec) {
        // four columns per thread (D % 4 == 0, 16-byte aligned bases)
        for (int c = threadIdx.x * 4; c < D; c += blockDim.x * 4) {
            float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int j = 0; j < k; ++j) {
                const long long row = place != nullptr ? place[t * k + j] : (long long)(t * k + j);
                if (row < 0) continue;
                const float4 v = load4(pair_out + (size_t)row * D + c);
                const float w = weight != nullptr ? weight[t * k + j] : 1.f;
                s.x = fmaf(w, v.x, s.x); s.y = fmaf(w, v.y, s.y); s.z = fmaf(w, v.z, s.z); s.w = fmaf(w, v.w, s.w);
            }
            if (shared != nullptr) {
                const float4 v = load4(shared + t * D + c);
                s.x = fmaf(gt, v.x, s.x); s.y = fmaf(gt, v.y, s.y); s.z = fmaf(gt, v.z, s.z); s.w = fmaf(gt, v.w, s.w);
            }
            *reinterpret_cast<float4*>(y + t * D + c) = s;
        }
        return;
    }
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
        float s = 0.f;
        for (int j = 0; j < k; ++j) {
            const long long row = place != nullptr ? place[t * k + j] : (long long)(t * k + j);
            if (row < 0) continue;
            const float v = to_float(pair_out[(size_t)row * D + c]);
            s = weight != nullptr ? fmaf(weight[t * k + j], v, s) : s + v;
        }
        if (shared != nullptr) s = fmaf(gt, to_float(shared[t * D + c]), s);
        y[t * D + c] = s;
    }
}

// out[i] = A[sorted[i] / a_div] (zeros where sorted[i] < 0): the left operand of the experts' first product in
// the order of `sorted`, for the tensor-core form that reads its tiles with TMA.  16-byte chunks.
__global__ void moe_gather_kernel(const uint4* __restrict__ A, int row_chunks, int a_div, const int* __restrict__ sorted,
                                  const int* __restrict__ n_tiles, int BM, int n_pairs, uint4* __restrict__ out) {
    const int i = blockIdx.x;
    if (i >= *n_tiles * BM) return;
    const int id = sorted[i];
    const bool ok = id >= 0 && id < n_pairs;
    const uint4* src = A + (size_t)(ok ? id / a_div : 0) * row_chunks;
    uint4* dst = out + (size_t)i * row_chunks;
    for (int c = threadIdx.x; c < row_chunks; c += blockDim.x) dst[c] = ok ? src[c] : make_uint4(0, 0, 0, 0);
}

template <int BM, bool GATED>
int launch_moe_bf16(const MoeGemm& p, int max_tiles, cudaStream_t stream) {
    auto kernel = moe_gemm_bf16_kernel<BM, GATED>;
    static bool attr_set[64] = {};
    int dev = 0;
    PL_CUDA(cudaGetDevice(&dev));
    PL_REQUIRE(dev >= 0 && dev < 64, "moe_gemm: device index %d is out of range", dev);
    if (!attr_set[dev]) {
        PL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, moe_gemm_smem<BM, GATED>()));
        attr_set[dev] = true;
    }
    kernel<<<dim3(max_tiles, (p.N + MG_BN - 1) / MG_BN), 128, moe_gemm_smem<BM, GATED>(), stream>>>(p);
    PL_LAUNCHED("moe_gemm_bf16");
    return 0;
}

}  // namespace

PL_EXPORT int pl_moe_topk(const float* z, int ldz, int tokens, int E, int k, int shared_gate, int* top_idx, float* top_w,
                          float* gate, cudaStream_t stream) {
    if (tokens == 0) return 0;
    PL_REQUIRE(tokens > 0 && E > 0 && k > 0 && k <= E && k <= 32 && E <= 1024 && ldz >= E + (shared_gate ? 1 : 0),
               "moe_topk: tokens=%d experts=%d top=%d (top <= 32, experts <= 1024)", tokens, E, k);
    moe_topk_kernel<<<(tokens + 3) / 4, 128, (size_t)4 * E * sizeof(float), stream>>>(z, ldz, tokens, E, k, shared_gate, top_idx,
                                                                                   top_w, gate);
    PL_LAUNCHED("moe_topk");
    return 0;
}

PL_EXPORT int pl_moe_sigmoid_topk(const float* z, int ldz, int tokens, int E, int k, int count, int keep, int group_top,
                                  int* top_idx, float* top_w, cudaStream_t stream) {
    if (tokens == 0) return 0;
    PL_REQUIRE(tokens > 0 && E > 0 && k > 0 && k <= E && E <= 1024 && ldz >= E, "moe_sigmoid_topk: tokens=%d experts=%d top=%d",
               tokens, E, k);
    PL_REQUIRE(count == 0 || (count > 0 && E % count == 0 && keep >= 1 && keep <= count && group_top >= 1 && group_top <= 8 &&
                              k <= E / count * keep),
               "moe_sigmoid_topk: %d groups of which %d stay, scored by their %d best (at most 8)", count, keep, group_top);
    moe_sigmoid_topk_kernel<<<(tokens + 3) / 4, 128, (size_t)4 * 3 * E * sizeof(float), stream>>>(z, ldz, tokens, E, k, count, keep,
                                                                                              group_top, top_idx, top_w);
    PL_LAUNCHED("moe_sigmoid_topk");
    return 0;
}

PL_EXPORT int pl_moe_align(const int* top_idx, int n_pairs, int E, int BM, int cap, int* sorted, int* tile_expert,
                           int* n_tiles, int* place, cudaStream_t stream) {
    PL_REQUIRE(n_pairs > 0 && E > 0 && E <= 1024 && (BM == 16 || BM == 64 || BM == 256) && cap % BM == 0,
               "moe_align: pairs=%d experts=%d BM=%d cap=%d", n_pairs, E, BM, cap);
    moe_align_kernel<<<1, 1024, 0, stream>>>(top_idx, n_pairs, E, BM, cap, sorted, tile_expert, n_tiles, place);
    PL_LAUNCHED("moe_align");
    return 0;
}

// out[cap][K] (bfloat16) = rows of A in the order of `sorted`; K a multiple of 8, both 16-byte aligned.
PL_EXPORT int pl_moe_gather(const void* A, int lda, int a_div, const int* sorted, const int* n_tiles, int BM, int cap,
                            int n_pairs, int K, void* out, cudaStream_t stream) {
    PL_REQUIRE(cap > 0 && K > 0 && K % 8 == 0 && lda == K && a_div > 0 && (((uintptr_t)A | (uintptr_t)out) & 15) == 0,
               "moe_gather: cap=%d K=%d lda=%d", cap, K, lda);
    moe_gather_kernel<<<cap, 128, 0, stream>>>((const uint4*)A, K / 8, a_div, sorted, n_tiles, BM, n_pairs, (uint4*)out);
    PL_LAUNCHED("moe_gather");
    return 0;
}

// gated != 0: out[pair][N] = act(A W_gate^T) * (A W_up^T) in `dtype`; else out[pair][N] = (A W^T) * row_scale in float32.
// BM is the tile height `sorted` was made for; tensor_cores != 0 asks for the mma.sync form (bfloat16, K % 8 == 0,
// lda % 8 == 0), which takes BM 16 or 64; the plain form takes BM 16 only.
PL_EXPORT int pl_moe_gemm(const void* A, int lda, int a_div, const void* W, void* out, int ldo, const int* sorted,
                          const int* tile_expert, const int* n_tiles, const float* row_scale, int n_pairs, int N, int K,
                          int gated, int act, float act_limit, int dtype, int BM, int max_tiles, int tensor_cores,
                          cudaStream_t stream) {
    PL_REQUIRE(n_pairs > 0 && N > 0 && K > 0 && a_div > 0 && max_tiles > 0, "moe_gemm: bad sizes");
    PL_REQUIRE(act >= 0 && act <= 2 && (act != 2 || act_limit > 0.f), "moe_gemm: unknown activation %d (limit %g)", act, act_limit);
    MoeGemm p = {A, W, out, sorted, tile_expert, n_tiles, row_scale, lda, a_div, ldo, n_pairs, N, K, act, act_limit};
    if (tensor_cores) {
        PL_REQUIRE(dtype == PL_BF16 && K % 8 == 0 && lda % 8 == 0 && ((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0,
                   "moe_gemm: the tensor-core form takes bfloat16 with K and lda multiples of 8");
        if (BM == 64) return gated ? launch_moe_bf16<64, true>(p, max_tiles, stream) : launch_moe_bf16<64, false>(p, max_tiles, stream);
        if (BM == 16) return gated ? launch_moe_bf16<16, true>(p, max_tiles, stream) : launch_moe_bf16<16, false>(p, max_tiles, stream);
        return pl_fail("moe_gemm: BM=%d", BM);
    }
    PL_REQUIRE(BM == 16, "moe_gemm: the plain form takes tiles of 16 pairs, not %d", BM);
    const dim3 grid(max_tiles, (N + 63) / 64);
    if (dtype == PL_F32) {
        if (gated) moe_gemm_plain_kernel<float, true><<<grid, 256, 0, stream>>>(p);
        else moe_gemm_plain_kernel<float, false><<<grid, 256, 0, stream>>>(p);
    } else if (dtype == PL_BF16) {
        if (gated) moe_gemm_plain_kernel<__nv_bfloat16, true><<<grid, 256, 0, stream>>>(p);
        else moe_gemm_plain_kernel<__nv_bfloat16, false><<<grid, 256, 0, stream>>>(p);
    } else {
        return pl_fail("moe_gemm: unknown dtype %d", dtype);
    }
    PL_LAUNCHED("moe_gemm_plain");
    return 0;
}

PL_EXPORT int pl_moe_combine(const void* pair_out, int pair_dtype, int k, const int* place, const float* weight,
                             const void* shared, int shared_dtype, const float* gate, float* y, int tokens, int D,
                             cudaStream_t stream) {
    if (tokens == 0) return 0;
    PL_REQUIRE(tokens > 0 && D > 0 && k > 0, "moe_combine: bad sizes");
    const int threads = D >= 1024 ? 256 : 128;
    const bool sf = shared == nullptr || shared_dtype == PL_F32;
    const int vec = D % 4 == 0 && (((uintptr_t)pair_out | (uintptr_t)shared | (uintptr_t)y) & 15) == 0;
    PL_REQUIRE(sf || shared_dtype == PL_BF16, "moe_combine: unknown dtype %d", shared_dtype);
    if (pair_dtype == PL_F32) {
        if (sf) moe_combine_kernel<float, float><<<tokens, threads, 0, stream>>>((const float*)pair_out, k, place, weight, (const float*)shared, gate, y, D, vec);
        else moe_combine_kernel<float, __nv_bfloat16><<<tokens, threads, 0, stream>>>((const float*)pair_out, k, place, weight, (const __nv_bfloat16*)shared, gate, y, D, vec);
    } else if (pair_dtype == PL_BF16) {
        if (sf) moe_combine_kernel<__nv_bfloat16, float><<<tokens, threads, 0, stream>>>((const __nv_bfloat16*)pair_out, k, place, weight, (const float*)shared, gate, y, D, vec);
        else moe_combine_kernel<__nv_bfloat16, __nv_bfloat16><<<tokens, threads, 0, stream>>>((const __nv_bfloat16*)pair_out, k, place, weight, (const __nv_bfloat16*)shared, gate, y, D, vec);
    } else {
        return pl_fail("moe_combine: unknown dtype %d", pair_dtype);
    }
    PL_LAUNCHED("moe_combine");
    return 0;
}
