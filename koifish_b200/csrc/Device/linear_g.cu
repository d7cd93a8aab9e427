// linear_g.cu -- matmuls of ANY shape over bf16 weights with fp32 results, for the layers whose sizes the tuned kernels of gemv.cu /
// gemm_tc.cu do not take (their K must be a multiple of 128 and their N of 16): y[m][n] = sum_k x[m][k] * W[n][k].
//   * activations x are bf16 bits (act_f32 = 0: the products are exact in fp32 and accumulate in fp32, i.e. the arithmetic of a bf16
//     tensor-core matmul) or float (act_f32 = 1: a true 32-bit matmul, FMA by FMA, no reduced-precision mode);
//   * "grouped" form for mixtures of experts: every output row (a slot) names the weight matrix it uses; slots of one expert are
//     contiguous (offsets[e] .. offsets[e+1]) and may gather their input row through src_row;
//   * DUAL form: two weight tables A, B of equal shape and y = silu(A x) * (B x), the gate / up pair of a gated feed-forward.
// Two kernels: a warp-per-output GEMV for a handful of rows (decode: every weight row is read once, 16-byte loads when the row length
// allows) and a 64 x 64 x 32 shared-memory tile kernel for panels (mma.sync m16n8k16 for bf16 activations, FFMA for float ones).
// No reference equivalent: the reference's SLP::Forw hands every shape to cuBLASLt (src/Device/CUDA/NeuronFuse.cu:305-381).
#include <algorithm>

#include "kf_common.cuh"

namespace {

struct LinArgs {
    const uint16_t* W0;          // single weight (dense) -- or
    const uint16_t* const* Wt0;  // table of per-expert weights (grouped)
    const uint16_t* W1;          // DUAL: second weight
    const uint16_t* const* Wt1;
    const void* x;               // [rows][ldx] bf16 bits or float
    void* y;                     // [slots][ldy] float (or, DUAL with out_act, the activation type)
    const int32_t* offsets;      // grouped: [E + 1] slot ranges; nullptr: one group [0, M)
    const int32_t* src_row;      // slot -> row of x; nullptr: slot
    const int32_t* slot_group;   // GEMV form: slot -> expert; nullptr: 0
    int M, N, K, ldx, ldy;
    int out_act;                 // DUAL or act != 0: 0 = float out, 1 = bf16 out, (float activations: float out)
    int act;                     // single-weight form: 0 = none, 1 = gelu (tanh form), 2 = relu squared, applied to the result
};
__device__ __forceinline__ float lin_act(float v, int act) {
    if (act == 1) return 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
    if (act == 2) return v > 0.f ? v * v : 0.f;
    return v;
}

template <typename TA>
__device__ __forceinline__ float ld_act(const TA* p);
template <>
__device__ __forceinline__ float ld_act<uint16_t>(const uint16_t* p) { return bf16_bits_to_f32(*p); }
template <>
__device__ __forceinline__ float ld_act<float>(const float* p) { return *p; }

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }

// ------------------------------------------------------------------------------------------------------------------ GEMV (few slots)
// one warp per (slot, output n): lanes stride over k, fixed butterfly reduction -> deterministic.
template <typename TA, bool DUAL>
__global__ void __launch_bounds__(256) kf_lin_gemv_kernel(LinArgs a) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n    = blockIdx.x * 8 + warp;
    const int slot = blockIdx.y;
    if (n >= a.N) return;
    const int g   = a.slot_group ? a.slot_group[slot] : 0;
    const int row = a.src_row ? a.src_row[slot] : slot;
    const uint16_t* w0 = (a.Wt0 ? a.Wt0[g] : a.W0) + (size_t)n * a.K;
    const uint16_t* w1 = DUAL ? (a.Wt1 ? a.Wt1[g] : a.W1) + (size_t)n * a.K : nullptr;
    const TA* x = (const TA*)a.x + (size_t)row * a.ldx;
    float s0 = 0.f, s1 = 0.f;
    const bool vec = (a.K % 8 == 0) && (a.ldx % 8 == 0) && (((uintptr_t)w0 & 15) == 0) && (((uintptr_t)x & 15) == 0) && (!DUAL || ((uintptr_t)w1 & 15) == 0);
    if (vec) {
        for (int k = lane * 8; k < a.K; k += 256) {
            const uint4 wv = *reinterpret_cast<const uint4*>(w0 + k);
            const uint32_t wq[4] = {wv.x, wv.y, wv.z, wv.w};
            float xv[8];
            if (sizeof(TA) == 2) {
                const uint4 xq4 = *reinterpret_cast<const uint4*>((const uint16_t*)x + k);
                const uint32_t xq[4] = {xq4.x, xq4.y, xq4.z, xq4.w};
#pragma unroll
                for (int j = 0; j < 4; j++) xv[2 * j] = bf16lo(xq[j]), xv[2 * j + 1] = bf16hi(xq[j]);
            } else {
                const float4 f0 = *reinterpret_cast<const float4*>((const float*)x + k), f1 = *reinterpret_cast<const float4*>((const float*)x + k + 4);
                xv[0] = f0.x, xv[1] = f0.y, xv[2] = f0.z, xv[3] = f0.w, xv[4] = f1.x, xv[5] = f1.y, xv[6] = f1.z, xv[7] = f1.w;
            }
#pragma unroll
            for (int j = 0; j < 4; j++) s0 = fmaf(bf16lo(wq[j]), xv[2 * j], s0), s0 = fmaf(bf16hi(wq[j]), xv[2 * j + 1], s0);
            if (DUAL) {
                const uint4 uv = *reinterpret_cast<const uint4*>(w1 + k);
                const uint32_t uq[4] = {uv.x, uv.y, uv.z, uv.w};
#pragma unroll
                for (int j = 0; j < 4; j++) s1 = fmaf(bf16lo(uq[j]), xv[2 * j], s1), s1 = fmaf(bf16hi(uq[j]), xv[2 * j + 1], s1);
            }
        }
    } else {
        for (int k = lane; k < a.K; k += 32) {
            const float xv = ld_act<TA>(x + k);
            s0 = fmaf(bf16_bits_to_f32(w0[k]), xv, s0);
            if (DUAL) s1 = fmaf(bf16_bits_to_f32(w1[k]), xv, s1);
        }
    }
    s0 = warp_sum(s0);
    if (DUAL) s1 = warp_sum(s1);
    if (lane == 0) {
        const float r = DUAL ? silu_f(s0) * s1 : lin_act(s0, a.act);
        if ((DUAL || a.act) && a.out_act == 1)
            ((uint16_t*)a.y)[(size_t)slot * a.ldy + n] = f32_to_bf16_bits(r);
        else
            ((float*)a.y)[(size_t)slot * a.ldy + n] = r;
    }
}

// ------------------------------------------------------------------------------------------------------------------ tile kernel
// 64 slots x 64 outputs per CTA, k in steps of 64 (bf16) or 32 (float); 256 threads.  Float activations: each thread a 4 x 4 block of FFMA accumulators.
// bf16 activations: 8 warps as 4 (m) x 2 (n), each warp 16 x 32 through mma.sync.m16n8k16; operands come from the same shared tiles.
// The next k step's operands are fetched into registers (16-byte loads when the row length and alignment allow, else element by
// element) while the current one is multiplied.  Every load is bounds-checked, so M, N and K are free.
constexpr int BM = 64, BN = 64;  // k step: 64 for bf16 activations (two 16-byte fetches per operand and thread in flight), 32 for float

__device__ __forceinline__ void mma_bf16_16816(float* c, const uint32_t* a, const uint32_t* b) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

__device__ __forceinline__ void ldsm_x4(uint32_t* r, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
// 8 consecutive k of one row: thread t fetches row t / 4, k offset (t % 4) * 8
template <typename T>
struct __align__(16) Frag8 {
    T v[8];
};
template <typename T>
__device__ __forceinline__ void fetch8(Frag8<T>& f, const T* base, size_t row_off, int k, int K, bool row_ok, bool vec) {
    if (row_ok && vec && k + 8 <= K) {
        if (sizeof(T) == 2) {
            *reinterpret_cast<uint4*>(f.v) = *reinterpret_cast<const uint4*>(base + row_off + k);
        } else {
            *reinterpret_cast<float4*>(f.v)     = *reinterpret_cast<const float4*>(base + row_off + k);
            *reinterpret_cast<float4*>(f.v + 4) = *reinterpret_cast<const float4*>(base + row_off + k + 4);
        }
        return;
    }
#pragma unroll
    for (int j = 0; j < 8; j++) f.v[j] = (row_ok && k + j < K) ? base[row_off + k + j] : T(0);
}

template <typename TA, bool DUAL>
__global__ void __launch_bounds__(256) kf_lin_tile_kernel(LinArgs a) {
    const int g    = blockIdx.z;
    const int lo   = a.offsets ? a.offsets[g] : 0;
    const int hi   = a.offsets ? a.offsets[g + 1] : a.M;
    const int n0 = blockIdx.x * BN;
    // a CTA walks the slot tiles blockIdx.y, blockIdx.y + gridDim.y, ... of its group: the grid is sized for the average group, not the worst
    for (int m0 = lo + blockIdx.y * BM; m0 < hi; m0 += gridDim.y * BM) {
    const uint16_t* W0 = a.Wt0 ? a.Wt0[g] : a.W0;
    const uint16_t* W1 = DUAL ? (a.Wt1 ? a.Wt1[g] : a.W1) : nullptr;
    constexpr bool MMA = sizeof(TA) == 2;
    constexpr int BK  = MMA ? 64 : 32, NF = BK / 32;
    constexpr int LDS = BK + 8;  // row pitch in elements: 16-byte aligned rows, conflict-free fragment loads
    __shared__ __align__(16) TA sx[BM][LDS];
    __shared__ __align__(16) uint16_t sw0[BN][LDS];
    __shared__ __align__(16) uint16_t sw1[DUAL ? BN : 1][LDS];
    const int tid = threadIdx.x;
    const int lr = tid >> 2, lk = (tid & 3) * 8;  // this thread's load: row lr, k offset lk
    int xrow = -1;
    {
        const int s = m0 + lr;
        if (s < hi) xrow = a.src_row ? a.src_row[s] : s;
    }
    const bool wok = n0 + lr < a.N;
    const size_t xoff = (size_t)(xrow < 0 ? 0 : xrow) * a.ldx, woff = (size_t)(n0 + lr) * a.K;
    const bool xvec = (a.ldx % 8 == 0) && (((uintptr_t)a.x & 15) == 0) && (a.K % 8 == 0);
    const bool wvec = (a.K % 8 == 0) && (((uintptr_t)W0 & 15) == 0) && (!DUAL || ((uintptr_t)W1 & 15) == 0);
    float acc0[16], acc1[DUAL ? 16 : 1];
#pragma unroll
    for (int i = 0; i < 16; i++) acc0[i] = 0.f;
    if (DUAL)
#pragma unroll
        for (int i = 0; i < 16; i++) acc1[i] = 0.f;
    const int warp = tid >> 5, lane = tid & 31;
    const int wm = warp & 3, wn = warp >> 2;      // MMA: warp tile rows wm*16, cols wn*32
    const int tr = tid >> 4, tc = tid & 15;        // FFMA: thread rows tr*4.., cols tc*4..
    Frag8<TA> fx[NF];
    Frag8<uint16_t> fw0[NF], fw1[NF];
    auto fetch = [&](int kb) {  // fragment f covers k = kb + f * 32 + lk .. + 7
#pragma unroll
        for (int f = 0; f < NF; f++) {
            fetch8<TA>(fx[f], (const TA*)a.x, xoff, kb + f * 32 + lk, a.K, xrow >= 0, xvec);
            fetch8<uint16_t>(fw0[f], W0, woff, kb + f * 32 + lk, a.K, wok, wvec);
            if (DUAL) fetch8<uint16_t>(fw1[f], W1, woff, kb + f * 32 + lk, a.K, wok, wvec);
        }
    };
    fetch(0);
    for (int k0 = 0; k0 < a.K; k0 += BK) {
        __syncthreads();  // the previous step's fragments have been read
#pragma unroll
        for (int f = 0; f < NF; f++) {
            const int kc = f * 32 + lk;
            if (MMA) {
                *reinterpret_cast<uint4*>(&sx[lr][kc]) = *reinterpret_cast<const uint4*>(fx[f].v);
            } else {
                *reinterpret_cast<float4*>(&sx[lr][kc])     = *reinterpret_cast<const float4*>(fx[f].v);
                *reinterpret_cast<float4*>(&sx[lr][kc + 4]) = *reinterpret_cast<const float4*>(fx[f].v + 4);
            }
            *reinterpret_cast<uint4*>(&sw0[lr][kc]) = *reinterpret_cast<const uint4*>(fw0[f].v);
            if (DUAL) *reinterpret_cast<uint4*>(&sw1[lr][kc]) = *reinterpret_cast<const uint4*>(fw1[f].v);
        }
        __syncthreads();
        if (k0 + BK < a.K) fetch(k0 + BK);  // next step's operands travel while this one is multiplied
        if (MMA) {
            // fragments through ldmatrix: A = 16 rows x 16 k of this warp's slots; B = two 8-output tiles per instruction
            const uint16_t* xa = (const uint16_t*)&sx[wm * 16][0];
#pragma unroll
            for (int kk = 0; kk < BK; kk += 16) {
                uint32_t af[4];
                ldsm_x4(af, xa + (lane & 15) * LDS + kk + (lane >> 4) * 8);
#pragma unroll
                for (int j = 0; j < 4; j += 2) {
                    const int nr = wn * 32 + j * 8 + (lane & 7) + (lane >> 4) * 8, kc = kk + ((lane >> 3) & 1) * 8;
                    uint32_t bf[4];
                    ldsm_x4(bf, &sw0[nr][kc]);
                    mma_bf16_16816(&acc0[j * 4], af, bf);
                    mma_bf16_16816(&acc0[(j + 1) * 4], af, bf + 2);
                    if (DUAL) {
                        ldsm_x4(bf, &sw1[nr][kc]);
                        mma_bf16_16816(&acc1[j * 4], af, bf);
                        mma_bf16_16816(&acc1[(j + 1) * 4], af, bf + 2);
                    }
                }
            }
        } else {
#pragma unroll 8
            for (int k = 0; k < BK; k++) {
                float xv[4], wv[4], uv[4];
#pragma unroll
                for (int i = 0; i < 4; i++) xv[i] = ld_act<TA>(&sx[tr * 4 + i][k]);
#pragma unroll
                for (int j = 0; j < 4; j++) wv[j] = bf16_bits_to_f32(sw0[tc * 4 + j][k]);
                if (DUAL)
#pragma unroll
                    for (int j = 0; j < 4; j++) uv[j] = bf16_bits_to_f32(sw1[tc * 4 + j][k]);
#pragma unroll
                for (int i = 0; i < 4; i++)
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        acc0[i * 4 + j] = fmaf(xv[i], wv[j], acc0[i * 4 + j]);
                        if (DUAL) acc1[i * 4 + j] = fmaf(xv[i], uv[j], acc1[i * 4 + j]);
                    }
            }
        }
    }
    auto store = [&](int r, int n, float v0, float v1) {
        const int s = m0 + r;
        if (s >= hi || n >= a.N) return;
        const float v = DUAL ? silu_f(v0) * v1 : lin_act(v0, a.act);
        if ((DUAL || a.act) && a.out_act == 1)
            ((uint16_t*)a.y)[(size_t)s * a.ldy + n] = f32_to_bf16_bits(v);
        else
            ((float*)a.y)[(size_t)s * a.ldy + n] = v;
    };
    if (MMA) {
        const int gr = lane >> 2, tg = lane & 3;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int n = n0 + wn * 32 + j * 8 + tg * 2, r = wm * 16 + gr;
            store(r, n, acc0[j * 4 + 0], DUAL ? acc1[j * 4 + 0] : 0.f);
            store(r, n + 1, acc0[j * 4 + 1], DUAL ? acc1[j * 4 + 1] : 0.f);
            store(r + 8, n, acc0[j * 4 + 2], DUAL ? acc1[j * 4 + 2] : 0.f);
            store(r + 8, n + 1, acc0[j * 4 + 3], DUAL ? acc1[j * 4 + 3] : 0.f);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) store(tr * 4 + i, n0 + tc * 4 + j, acc0[i * 4 + j], DUAL ? acc1[i * 4 + j] : 0.f);
    }
    __syncthreads();  // the shared tiles are free for the next slot tile
    }
}

template <typename TA, bool DUAL>
int launch(kf_ctx* ctx, const LinArgs& a, int slots, int groups, bool gemv) {
    if (gemv) {
        dim3 grid((a.N + 7) / 8, slots);
        kf_lin_gemv_kernel<TA, DUAL><<<grid, 256, 0, ctx->stream>>>(a);
    } else {
        const int tiles = (slots + BM - 1) / BM;
        const int gy    = groups > 1 ? std::min(tiles, std::max(1, (2 * slots / groups + BM - 1) / BM)) : tiles;
        dim3 grid((a.N + BN - 1) / BN, gy, groups);
        kf_lin_tile_kernel<TA, DUAL><<<grid, 256, 0, ctx->stream>>>(a);
    }
    KF_LAUNCH_CHECK(ctx);
    return KF_OK;
}
int dispatch(kf_ctx* ctx, const LinArgs& a, int slots, int groups, bool gemv, bool dual, int act_f32) {
    if (act_f32) return dual ? launch<float, true>(ctx, a, slots, groups, gemv) : launch<float, false>(ctx, a, slots, groups, gemv);
    return dual ? launch<uint16_t, true>(ctx, a, slots, groups, gemv) : launch<uint16_t, false>(ctx, a, slots, groups, gemv);
}
constexpr int kGemvMaxSlots = 16;
}  // namespace

extern "C" int kf_linear_g(kf_ctx* ctx, float* y, int ldy, const kf_tensor_desc* w, const void* x, int act_f32, int ldx, int M) {
    if (!ctx || !y || !w || !x) return KF_ERR_BAD_ARG;
    KF_REQUIRE(ctx, w->type == KF_T_BF16 && M >= 1 && w->rows >= 1 && w->cols >= 1 && ldx >= w->cols && ldy >= w->rows, "bf16 weight, ld >= extent");
    // few outputs over a long reduction (a gate or a router of a panel): tiles would leave all but a handful of SMs idle, so every
    // (token, output) pair gets a warp instead; the weight (<= 64 rows) stays in L2
    const bool skinny = w->rows <= 64 && w->cols >= 512 && M > kGemvMaxSlots;
    // shapes the tuned kernels take go there (tcgen05 / TMEM panels, the HBM-rate GEMV); fp32 result through their fp32 epilogue
    if (!skinny && !act_f32 && ldx == w->cols && ldy == w->rows && w->cols % 128 == 0 && w->rows % 16 == 0 && w->rows >= 16 && ctx->tc_min_m != 0 &&
        (((uintptr_t)w->data_dev | (uintptr_t)x | (uintptr_t)y) & 15) == 0)
        return kf_linear(ctx, y, w, x, M, KF_EPI_F32, nullptr);
    LinArgs a = {};
    a.W0 = (const uint16_t*)w->data_dev, a.x = x, a.y = y, a.M = M, a.N = w->rows, a.K = w->cols, a.ldx = ldx, a.ldy = ldy;
    return dispatch(ctx, a, M, 1, M <= kGemvMaxSlots || skinny, false, act_f32);
}
// y = silu(Wg x) * (Wu x), written in the activation type (bf16 bits, or float when act_f32)
extern "C" int kf_linear_g_swiglu(kf_ctx* ctx, void* y, int ldy, const kf_tensor_desc* wg, const kf_tensor_desc* wu, const void* x, int act_f32,
                                  int ldx, int M) {
    if (!ctx || !y || !wg || !wu || !x) return KF_ERR_BAD_ARG;
    KF_REQUIRE(ctx, wg->type == KF_T_BF16 && wu->type == KF_T_BF16 && wg->rows == wu->rows && wg->cols == wu->cols && M >= 1 && ldx >= wg->cols &&
                        ldy >= wg->rows, "gate / up: bf16, equal shapes");
    LinArgs a = {};
    a.W0 = (const uint16_t*)wg->data_dev, a.W1 = (const uint16_t*)wu->data_dev, a.x = x, a.y = y, a.M = M, a.N = wg->rows, a.K = wg->cols;
    a.ldx = ldx, a.ldy = ldy, a.out_act = act_f32 ? 0 : 1;
    return dispatch(ctx, a, M, 1, M <= kGemvMaxSlots, true, act_f32);
}
// Grouped matmul over expert-sorted slots.  w_table / w2_table: device arrays of n_groups bf16 weight pointers ([N][K] each);
// offsets: device int32 [n_groups + 1]; slot_group: device int32 [slots] (the expert of each slot); src_row: device int32 [slots] or
// NULL.  w2_table != NULL: y = silu(W x) * (W2 x) in the activation type; else y is float.  `slots` is the launch bound (tokens x top).
extern "C" int kf_linear_grouped(kf_ctx* ctx, void* y, int ldy, const void* const* w_table, const void* const* w2_table, int n_groups, int N, int K,
                                 const void* x, int act_f32, int ldx, const int32_t* offsets, const int32_t* slot_group, const int32_t* src_row,
                                 int slots) {
    if (!ctx || !y || !w_table || !x || !offsets || !slot_group) return KF_ERR_BAD_ARG;
    KF_REQUIRE(ctx, n_groups >= 1 && N >= 1 && K >= 1 && slots >= 1 && ldx >= K && ldy >= N, "shape");
    LinArgs a = {};
    a.Wt0 = (const uint16_t* const*)w_table, a.Wt1 = (const uint16_t* const*)w2_table, a.x = x, a.y = y, a.M = slots, a.N = N, a.K = K;
    a.ldx = ldx, a.ldy = ldy, a.offsets = offsets, a.slot_group = slot_group, a.src_row = src_row, a.out_act = act_f32 ? 0 : 1;
    return dispatch(ctx, a, slots, n_groups, slots <= kGemvMaxSlots, w2_table != nullptr, act_f32);
}

// The single-weight grouped form with an activation on the result (1: gelu, tanh form; 2: relu squared), written in the activation type
// (bf16 bits, or float when act_f32): the up projection of experts that have no gate.  act 0 = kf_linear_grouped without a second table.
extern "C" int kf_linear_grouped_act(kf_ctx* ctx, void* y, int ldy, const void* const* w_table, int n_groups, int N, int K, const void* x, int act_f32, int ldx,
                                     const int32_t* offsets, const int32_t* slot_group, const int32_t* src_row, int slots, int act) {
    if (!ctx || !y || !w_table || !x || !offsets || !slot_group) return KF_ERR_BAD_ARG;
    KF_REQUIRE(ctx, n_groups >= 1 && N >= 1 && K >= 1 && slots >= 1 && ldx >= K && ldy >= N && act >= 0 && act <= 2, "shape / act");
    LinArgs a = {};
    a.Wt0 = (const uint16_t* const*)w_table, a.x = x, a.y = y, a.M = slots, a.N = N, a.K = K;
    a.ldx = ldx, a.ldy = ldy, a.offsets = offsets, a.slot_group = slot_group, a.src_row = src_row, a.out_act = act_f32 ? 0 : 1, a.act = act;
    return dispatch(ctx, a, slots, n_groups, slots <= kGemvMaxSlots, false, act_f32);
}
