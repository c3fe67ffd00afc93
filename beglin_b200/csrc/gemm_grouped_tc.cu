// The experts' products of a routed feed-forward on the fifth-generation tensor cores:
//   out[row, n] = act(sum_k X[row, k] * W[e][n, k])     for the rows offsets[e] .. offsets[e + 1] of expert e,
// bfloat16 X and W, float accumulation.  The main loop is that of the plain tcgen05 product (gemm_tcgen05.cu): operand tiles
// by TMA (128-byte swizzle), one thread issues tcgen05.mma with the accumulator in tensor memory, four warps read it back
// with tcgen05.ld.  The weights are the M side (128 output features of ONE expert per CTA), the rows the N side (BN of them).
//
// What is grouped about it: the experts' matrices lie one behind the other, [E * n_out, K], under one tensor map, and the
// rows, sorted by expert, under another.  Which expert a CTA serves is not known when the kernel is launched (the tokens are
// routed on the device): the grid has a row tile for every tile that any distribution of the rows could need, a CTA looks
// its expert and rows up in `offsets` first, and one without rows frees its columns of tensor memory and returns.  A tile whose box
// runs past its expert's rows (or features) reads the neighbour's; those columns (or lanes) of the accumulator are not stored.
//
// Every wait on an mbarrier is bounded: when one runs out the thread records BG_STATUS_TIMEOUT and the CTA winds down
// (tensor memory is freed).
#include "tc_common.cuh"

namespace bg {

struct GroupedTcParams {
    void* out;              // [rows][ldo] float or bfloat16
    int ldo, out_dtype;
    int n_out, K, E;
    int act;                // 0: none; 1: the square of relu
    const int* offsets;     // [E + 1]
    unsigned* status;
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(TC_THREADS)
gemm_grouped_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, GroupedTcParams p) {
    constexpr unsigned A_BYTES = TC_BM * TC_BK * 2;
    constexpr unsigned B_BYTES = BN * TC_BK * 2;
    constexpr unsigned STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr unsigned TMEM_COLS = BN < 32 ? 32 : BN;
    extern __shared__ unsigned char gtc_smem_raw[];
    unsigned char* tiles = (unsigned char*)(((uintptr_t)gtc_smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) unsigned long long full_bar[STAGES];
    __shared__ __align__(8) unsigned long long empty_bar[STAGES];
    __shared__ __align__(8) unsigned long long acc_bar;
    __shared__ unsigned tmem_base_sh;
    __shared__ int failed;
    __shared__ int where[3];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile_m = blockIdx.x;
    const int n_kb = (p.K + TC_BK - 1) / TC_BK;

    // Tensor memory is asked for at once, before the wait for the kernel ahead, as in every kernel of this library that
    // holds any: a CTA that waited for its predecessor first could find the columns taken by CTAs of a successor that
    // wait for this kernel to end.
    pdl_launch();
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        mbar_init(&acc_bar, 1);
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(&tmem_base_sh)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    pdl_wait();                                   // the offsets are this step's
    if (threadIdx.x == 0) {
        int e = -1, r0 = 0, n = 0, before = 0;
        for (int i = 0; i < p.E; ++i) {
            const int lo = p.offsets[i], cnt = p.offsets[i + 1] - lo;
            const int t = (cnt + BN - 1) / BN;
            if ((int)blockIdx.y < before + t) { e = i; r0 = lo + ((int)blockIdx.y - before) * BN; n = min(BN, lo + cnt - r0); break; }
            before += t;
        }
        where[0] = e; where[1] = r0; where[2] = n;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = tmem_base_sh;
    const int e = where[0], row0 = where[1], n_rows = where[2];     // e < 0: a CTA without rows only frees its columns
    const int w_row = e * p.n_out + tile_m * TC_BM;

    if (e < 0) {
    } else if (warp == 0) {
        if (lane == 0) {
            for (int i = 0; i < n_kb; ++i) {
                const int s = i % STAGES;
                if (i >= STAGES && !mbar_wait(&empty_bar[s], ((i / STAGES) - 1) & 1)) { atomicExch(&failed, 1); break; }
                unsigned char* a = tiles + (size_t)s * STAGE_BYTES;
                mbar_expect_tx(&full_bar[s], STAGE_BYTES);
                tma_load_2d(a, &map_w, i * TC_BK, w_row, &full_bar[s]);
                tma_load_2d(a + A_BYTES, &map_x, i * TC_BK, row0, &full_bar[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr unsigned idesc = instr_desc_bf16(TC_BM, BN < 16 ? 16 : BN);
            for (int i = 0; i < n_kb; ++i) {
                const int s = i % STAGES;
                if (!mbar_wait(&full_bar[s], (i / STAGES) & 1)) { atomicExch(&failed, 1); break; }
                tc_fence_after();
                const unsigned a_addr = smem_u32(tiles + (size_t)s * STAGE_BYTES);
                const unsigned b_addr = a_addr + A_BYTES;
#pragma unroll
                for (int k = 0; k < TC_BK / 16; ++k)
                    tc_mma(tmem_base, smem_desc_sw128(a_addr + k * 32), smem_desc_sw128(b_addr + k * 32), idesc, (i > 0 || k > 0) ? 1u : 0u);
                tc_commit(&empty_bar[s]);
            }
            tc_commit(&acc_bar);
        }
    } else {
        // warps 2..5 own tensor-memory lanes 32 * (warp % 4) .. + 31: a lane is an output feature, a column a row
        const int quarter = warp & 3;
        const int m = tile_m * TC_BM + quarter * 32 + lane;
        bool ok = mbar_wait(&acc_bar, 0);
        if (!ok) atomicExch(&failed, 1);
        tc_fence_after();
        if (ok) {
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                if (c >= n_rows) break;                                  // warp-uniform
                unsigned r[16];
                tc_ld16(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)c, r);
                if (m < p.n_out) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        if (c + j >= n_rows) break;
                        float v = __uint_as_float(r[j]);
                        if (p.act == 1) { v = fmaxf(v, 0.0f); v *= v; }
                        const size_t o = (size_t)(row0 + c + j) * p.ldo + m;
                        if (p.out_dtype == BG_DTYPE_F32) ((float*)p.out)[o] = v;
                        else ((__nv_bfloat16*)p.out)[o] = __float2bfloat16_rn(v);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && failed && p.status) atomicOr(p.status, BG_STATUS_TIMEOUT);
}

template <int BN, int STAGES>
static int grouped_launch(const CUtensorMap& mw, const CUtensorMap& mx, const GroupedTcParams& p, int rows, cudaStream_t stream) {
    auto kern = gemm_grouped_tcgen05_kernel<BN, STAGES>;
    size_t smem = (size_t)STAGES * (TC_BM * TC_BK * 2 + BN * TC_BK * 2) + 1024;
    static bool set = false;
    if (!set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        set = true;
    }
    const int row_tiles = rows / BN + p.E;
    if (row_tiles > 65535) return BG_ERR_SHAPE;
    dim3 grid((p.n_out + TC_BM - 1) / TC_BM, row_tiles);
    launch(kern, grid, dim3(TC_THREADS), smem, stream, mw, mx, p);
    BG_LAUNCH_CHECK();
    return BG_OK;
}

}  // namespace bg

using namespace bg;

// X [rows, K] bfloat16 (row stride ldx), W [E * n_out, K] bfloat16 (row stride ldw; expert e's rows start at e * n_out),
// out [rows, ldo] float or bfloat16.  Strides multiples of 8, bases 16-byte aligned.
extern "C" int bg_gemm_grouped_tc(const void* W, int E, int n_out, int K, int ldw, const void* X, int rows, int ldx, void* out,
                                  int out_dtype, int ldo, const int* offsets, int act, unsigned* status, cudaStream_t stream) {
    if (rows <= 0 || n_out <= 0) return BG_OK;
    if (K <= 0 || E <= 0) return BG_ERR_SHAPE;
    if ((ldw % 8) || (ldx % 8) || ((uintptr_t)W % 16) || ((uintptr_t)X % 16)) return BG_ERR_ALIGN;
    if (out_dtype != BG_DTYPE_F32 && out_dtype != BG_DTYPE_BF16) return BG_ERR_DTYPE;
    GroupedTcParams p;
    p.out = out; p.ldo = ldo; p.out_dtype = out_dtype; p.n_out = n_out; p.K = K; p.E = E; p.act = act; p.offsets = offsets;
    p.status = status;
    // rows per tile from the rows an expert gets on average: the shapes of the step alone decide
    const int avg = (rows + E - 1) / E;
    const int bn = avg <= 16 ? 16 : avg <= 32 ? 32 : avg <= 64 ? 64 : avg <= 128 ? 128 : 256;
    CUtensorMap mw, mx;
    int rc = weight_map(&mw, W, E * n_out, K, ldw);
    if (rc != BG_OK) return rc;
    rc = make_map(&mx, X, rows, K, ldx, bn);
    if (rc != BG_OK) return rc;
    switch (bn) {
        case 16: return grouped_launch<16, 4>(mw, mx, p, rows, stream);
        case 32: return grouped_launch<32, 4>(mw, mx, p, rows, stream);
        case 64: return grouped_launch<64, 4>(mw, mx, p, rows, stream);
        case 128: return grouped_launch<128, 3>(mw, mx, p, rows, stream);
        default: {
            // many rows: bound by the tensor cores.  With more CTAs than SMs, two stages keep a CTA under half of an SM's
            // shared memory, so that two CTAs share the SM and one's epilogue runs under the other's MMAs.
            const long long ctas = (long long)((n_out + TC_BM - 1) / TC_BM) * (rows / 256 + E);
            if (ctas > sm_count()) return grouped_launch<256, 2>(mw, mx, p, rows, stream);
            return grouped_launch<256, 4>(mw, mx, p, rows, stream);
        }
    }
}
