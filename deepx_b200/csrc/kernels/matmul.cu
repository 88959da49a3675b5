// dx_matmul: batched row-major C[b,M,N] = A[b,M,K] · B[b,K,N].
//
// bf16 / f16: persistent, warp-specialised tcgen05 kernels (sm_100a).
//   * one CTA per SM walks output tiles of 128 × 256 (or 128 × 128 / 128 × 64 when the matrix gives
//     too few wide tiles; a pair of CTAs shares 256 × 256 tiles when there are enough of those);
//   * warp 0 (one elected lane) is the TMA producer: per 64-deep K block it loads an
//     A tile (128 rows × 64 K, K-major) and four B tiles (64 K × 64 N, N-major) into a
//     shared-memory ring with 128-byte swizzle, completing on an mbarrier;
//   * warp 1 (one elected lane) issues tcgen05.mma (M128 N256 K16, kind::f16, fp32
//     accumulate) four times per stage, reading operands straight from shared memory
//     through matrix descriptors; tcgen05.commit releases the stage / publishes the tile;
//   * accumulators live in TMEM, double-buffered (2 × 256 columns), so the epilogue of
//     tile i overlaps the main loop of tile i+1;
//   * warps 2-9 are the epilogue, two per TMEM lane quarter: tcgen05.ld, round fp32 → 16-bit
//     once, turn 32 × 64 blocks round in shared memory, store whole 128-byte lines of C.
// Matrices with few rows take cluster kernels that split K (one row of 128 × 64 tiles, or a few
// rows of 256 × 256 pair tiles) and combine the partial tiles through distributed shared memory.
// B is consumed in its natural [K,N] layout (MN-major operand), so no transpose pass.
// No cluster launch and no multicast: every CTA loads its own tiles; A and B fit in L2.
//
// Every wait on an mbarrier is bounded by a clock: on expiry the kernel records a code in
// a status word, all roles leave their loops, TMEM is freed and the kernel returns; the
// host turns the status into DX_E_CUDA.
//
// f32 / f64: a register-tiled SIMT FMA kernel (the reference calls cuBLAS Sgemm/Dgemm,
// executor/op-cuda/src/deepx/tensorfunc/matmul_cublas.hpp:16-145; a 1e-5 bound rules out
// plain TF32 tensor-core math).
#include <cuda.h>

#include <cstdlib>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace dx {
namespace {

// ---- tile configuration ----------------------------------------------------------------
constexpr int BM = 128, BN = 256, BK = 64;   // CTA tile; BK·2 bytes = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int ACC_STAGES = 2;
constexpr int NUM_THREADS = 192;             // TMA warp, MMA warp, 4 epilogue warps (the split-K kernels)
constexpr int G_THREADS = 320;               // TMA warp, MMA warp, 8 epilogue warps (the persistent tile kernels)
constexpr int A_STAGE_BYTES = BM * BK * 2;   // 16 KiB
constexpr int B_BOX_N = 64;                  // one TMA box of B: 64 K-rows × 64 N (128 bytes wide)
constexpr int B_BOX_BYTES = BK * B_BOX_N * 2;  // 8 KiB
constexpr int B_STAGE_BYTES = B_BOX_BYTES * (BN / B_BOX_N);  // 32 KiB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
constexpr int TMEM_COLS = ACC_STAGES * BN;   // 512
constexpr long long WAIT_LIMIT_CYCLES = 4000000000ll;  // ~2 s

enum GemmStatus : int { GEMM_OK = 0, GEMM_TIMEOUT_FULL = 1, GEMM_TIMEOUT_EMPTY = 2, GEMM_TIMEOUT_TMEM_FULL = 3,
                        GEMM_TIMEOUT_TMEM_EMPTY = 4 };

// ---- PTX wrappers -------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false when the clock limit passed or another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > WAIT_LIMIT_CYCLES) return false;
    }
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap *map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives on the mbarrier once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- descriptors ----------------------------------------------------------------------------
// Shared-memory matrix descriptor (64-bit): start address >>4 in [0,14), leading byte offset >>4
// in [16,30), stride byte offset >>4 in [32,46), descriptor version 1 in [46,48), swizzle mode in
// [61,64) (2 = 128-byte swizzle of 16-byte chunks, 1 = 128-byte swizzle of 32-byte chunks).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                                   uint32_t swizzle_mode = 2) {
    uint64_t d = 0;
    d |= uint64_t((saddr >> 4) & 0x3FFF);
    d |= uint64_t((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= uint64_t((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= uint64_t(1) << 46;
    d |= uint64_t(swizzle_mode) << 61;
    return d;
}
// Instruction descriptor (32-bit) for kind::f16: D format [4,6) 1 = f32; A format [7,10), B format
// [10,13) (0 = f16, 1 = bf16); A major bit 15, B major bit 16 (0 = K-major, 1 = MN-major);
// N>>3 in [17,23); M>>4 in [24,29).
__host__ __device__ constexpr uint32_t make_idesc_n(int ab_format, int n) {
    return (1u << 4) | (uint32_t(ab_format) << 7) | (uint32_t(ab_format) << 10) | (0u << 15) | (1u << 16) |
           (uint32_t(n >> 3) << 17) | (uint32_t(BM >> 4) << 24);
}

// Tile order.  The CTAs that run at the same time take consecutive tile numbers, so the order decides
// what they share in L2.  Rows of tiles are taken in groups of RASTER_GROUP: inside a group the order
// is column by column, so one wave covers a few columns of B against the SAME group of A row-panels
// (8 panels of A stay hot while B streams past) instead of every A panel against two columns of B.
__device__ __forceinline__ void grouped_tile_coords(int tile, int tiles_m, int tiles_n, int RASTER_GROUP, int &b, int &tm, int &tn) {
    const int per_batch = tiles_m * tiles_n;
    b = tile / per_batch;
    const int t = tile - b * per_batch;
    const int group_tiles = RASTER_GROUP * tiles_n;
    const int g = t / group_tiles;
    const int first_m = g * RASTER_GROUP;
    const int gm = min(tiles_m - first_m, RASTER_GROUP);
    const int r = t - g * group_tiles;
    tn = r / gm;
    tm = first_m + (r - tn * gm);
}

// ---- the way out: TMEM → registers → C ----------------------------------------------------------
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}

template <typename T> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<bf16>(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<f16>(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}

constexpr int EPI_ROWS = 32, EPI_COLS = 64;              // one block: a warp's 32 rows × 64 columns
constexpr int EPI_WARP_BYTES = EPI_ROWS * EPI_COLS * 2;  // 4 KiB per epilogue warp, 128 bytes per row
constexpr int EPI_BYTES = 8 * EPI_WARP_BYTES;            // 32 KiB for the eight epilogue warps

// One epilogue warp drains its 32 rows of a finished accumulator (`width` columns at `tmem_acc`),
// rounding fp32 to the 16-bit type once.  Out of TMEM a lane holds one ROW; stored like that, one
// store instruction touches 32 different rows, 16 bytes each.  So when C allows 16-byte stores
// (`staged`: base and pitch multiples of 16 bytes) the warp turns each block of 32 rows × 64 columns
// round in its own 4 KiB of shared memory — rows of 128 bytes, the 16-byte chunks of a row
// XOR-swizzled by the row number so that both directions are free of bank conflicts — and writes it
// out with eight lanes per row: every store instruction covers four whole 128-byte lines of C.
// (A TMA store of the same block costs the issuing lane about 300 cycles per 4 KiB, measured, and the
// wait before its buffer may be reused another 200; the plain stores need neither.)
// Without `staged` each lane stores its own row from registers.
// The second half of the way out: a warp's block of 32 rows × 64 columns, one row per lane in r[2][32] as fp32 bit
// patterns, rounded once and written to C (turned round in shared memory when `staged`, else row by row).
template <typename T>
__device__ __forceinline__ void emit_block(const uint32_t (&r)[2][32], T *C, bool staged, uint32_t stage_smem, int M, int N, int b, int row0,
                                           int col, int lane) {
    const int row = row0 + lane;
    if (row0 >= M || col >= N) return;  // the whole block lies outside C (same answer in every lane)
    if (staged) {
        const uint32_t mine = stage_smem + lane * 128;
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                const int chunk = h * 4 + v;
                st_shared_v4(mine + ((chunk ^ (lane & 7)) << 4),
                             pack2<T>(__uint_as_float(r[h][8 * v + 0]), __uint_as_float(r[h][8 * v + 1])),
                             pack2<T>(__uint_as_float(r[h][8 * v + 2]), __uint_as_float(r[h][8 * v + 3])),
                             pack2<T>(__uint_as_float(r[h][8 * v + 4]), __uint_as_float(r[h][8 * v + 5])),
                             pack2<T>(__uint_as_float(r[h][8 * v + 6]), __uint_as_float(r[h][8 * v + 7])));
            }
        __syncwarp();
        // lane → (row lane/8 of a group of four rows, chunk lane%8): 4 rows × 128 bytes per instruction
        const int chunk = lane & 7;
        const int gcol = col + chunk * 8;
        uint4 v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int rr = i * 4 + (lane >> 3);
            v[i] = ld_shared_v4(stage_smem + rr * 128 + ((chunk ^ (rr & 7)) << 4));
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int rr = i * 4 + (lane >> 3);
            if (row0 + rr < M && gcol < N) *reinterpret_cast<uint4 *>(C + (size_t(b) * M + row0 + rr) * N + gcol) = v[i];
        }
        __syncwarp();  // the block is in registers / on its way before the next one overwrites the buffer
    } else if (row < M) {
        T *crow = C + (size_t(b) * M + row) * N;
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (col + 32 * h + j < N) crow[col + 32 * h + j] = from_compute<T>(__uint_as_float(r[h][j]));
    }
}

template <typename T>
__device__ __forceinline__ void drain_accumulator(uint32_t tmem_acc, int width, T *C, bool staged, uint32_t stage_smem, int M, int N,
                                                  int b, int row0, int col0, int lane) {
#pragma unroll 1
    for (int c0 = 0; c0 < width; c0 += EPI_COLS) {
        uint32_t r[2][32];
        tmem_ld_32x32b_x32(tmem_acc + c0, r[0]);
        tmem_ld_32x32b_x32(tmem_acc + c0 + 32, r[1]);
        tmem_ld_wait();
        emit_block<T>(r, C, staged, stage_smem, M, N, b, row0, col0 + c0, lane);
    }
}

// Tile width BN_ (256, 128 or 64 columns) is chosen by the host from how many tiles each width
// gives: a narrow tile has a worse ratio of shared-memory reads to math, but 128 × 256 tiles of a
// matrix with few rows leave most SMs without work.  Narrower tiles take a deeper ring.
template <int BN_> struct TileCfg {
    static constexpr int B_STAGE = B_BOX_BYTES * (BN_ / B_BOX_N);
    static constexpr int STAGE = A_STAGE_BYTES + B_STAGE;
    static constexpr int NSTAGES = (192 * 1024) / STAGE;  // 4, 6, 8
    static constexpr int RING = NSTAGES * STAGE;
    static constexpr int SMEM = RING + EPI_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
    static constexpr int TMEM = ACC_STAGES * BN_;
};
static_assert(TileCfg<256>::SMEM <= 227 * 1024 && TileCfg<128>::SMEM <= 227 * 1024 && TileCfg<64>::SMEM <= 227 * 1024, "shared memory");

struct GemmParams {
    int M, N, K, batch;
    int tiles_m, tiles_n, num_tiles, k_blocks;
    int raster;   // rows of tiles per raster group
    int c_staged; // C takes 16-byte stores (base and pitch multiples of 16 bytes): blocks are turned round in shared memory
    int *status;
};

template <typename T, int BN_>
__global__ void __launch_bounds__(G_THREADS, 1)
    gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, T *__restrict__ C,
                        GemmParams p) {
    using Cfg = TileCfg<BN_>;
    constexpr int NS = Cfg::NSTAGES;
    // A lane quarter of TMEM is reachable from warps with the same warp % 4 only: two warps per quarter, each
    // taking half of the tile's columns (a 64-column tile has one 64-column block per quarter: four warps work).
    constexpr int EPI_WARPS = BN_ >= 128 ? 8 : 4;
    constexpr int EPI_WIDTH = BN_ >= 128 ? BN_ / 2 : BN_;
    extern __shared__ uint8_t smem_raw[];
    // 128-byte swizzle atoms are 1024 bytes: stage bases must be 1024-byte aligned
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t epi_smem = smem_base + Cfg::RING;
    constexpr int BAR_OFF = Cfg::RING + EPI_BYTES;
    const uint32_t bars = smem_base + BAR_OFF;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (NS + s); };
    auto tfull_bar = [&](int a) { return bars + 8u * (2 * NS + a); };
    auto tempty_bar = [&](int a) { return bars + 8u * (2 * NS + ACC_STAGES + a); };
    constexpr int SLOT_OFF = 8 * (2 * NS + 2 * ACC_STAGES);
    const uint32_t tmem_slot = bars + SLOT_OFF;
    uint8_t *gen_base = smem_raw + (smem_base - smem_u32(smem_raw));
    volatile uint32_t *tmem_slot_ptr = reinterpret_cast<volatile uint32_t *>(gen_base + BAR_OFF + SLOT_OFF);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(gen_base + BAR_OFF + SLOT_OFF + 8);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < ACC_STAGES; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), EPI_WARPS);  // one arrival per working epilogue warp
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
    }
    if (warp == 1) tmem_alloc(tmem_slot, Cfg::TMEM);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_ptr;

    if (warp == 0) {
        // ===== TMA producer =====
        if (lane == 0) {
            griddep_wait();  // the one thread that first touches global memory; every other role follows its loads
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
                int b, tm, tn;
                grouped_tile_coords(tile, p.tiles_m, p.tiles_n, p.raster, b, tm, tn);
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1, abort_flag)) {
                        if (!*abort_flag) { *abort_flag = 1; atomicExch(p.status, GEMM_TIMEOUT_EMPTY); }
                        ok = false;
                        break;
                    }
                    const uint32_t sa = smem_base + stage * Cfg::STAGE;
                    const uint32_t sb = sa + A_STAGE_BYTES;
                    mbar_expect_tx(full_bar(stage), Cfg::STAGE);
                    tma_load_3d(sa, &tmap_a, full_bar(stage), kb * BK, tm * BM, b);
#pragma unroll
                    for (int j = 0; j < BN_ / B_BOX_N; ++j)
                        tma_load_3d(sb + j * B_BOX_BYTES, &tmap_b, full_bar(stage), tn * BN_ + j * B_BOX_N, kb * BK, b);
                    if (++stage == NS) { stage = 0; phase ^= 1; }
                }
            }
            if (*abort_flag) {
                // give copies already in flight time to land before the CTA's shared memory is released
                const long long t0 = clock64();
                while (clock64() - t0 < 2000000ll) {}
            }
        }
    } else if (warp == 1) {
        // ===== MMA issuer =====
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_n(std::is_same<T, bf16>::value ? 1 : 0, BN_);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
                if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1, abort_flag)) {
                    if (!*abort_flag) { *abort_flag = 1; atomicExch(p.status, GEMM_TIMEOUT_TMEM_EMPTY); }
                    break;
                }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + acc * BN_;
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
                        if (!*abort_flag) { *abort_flag = 1; atomicExch(p.status, GEMM_TIMEOUT_FULL); }
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sa = smem_base + stage * Cfg::STAGE;
                    const uint32_t sb = sa + A_STAGE_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // A: K-major, 8-row groups 1024 bytes apart; step 16 K elements = 32 bytes inside the swizzle row
                        const uint64_t adesc = make_smem_desc(sa + k * (UMMA_K * 2), 16, 1024);
                        // B: N-major, 64-column panels 8192 bytes apart (LBO), 8-K-row groups 1024 bytes apart (SBO);
                        // step 16 K rows = 2048 bytes
                        const uint64_t bdesc = make_smem_desc(sb + k * (UMMA_K * 128), B_BOX_BYTES, 1024);
                        umma_f16(tmem_d, adesc, bdesc, idesc, (kb | k) != 0);
                    }
                    umma_commit(empty_bar(stage));  // stage reusable once these MMAs have read it
                    if (++stage == NS) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                umma_commit(tfull_bar(acc));  // accumulator complete
                if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1; }
            }
        }
    } else if (warp - 2 < EPI_WARPS) {
        // ===== epilogue: warps 2..9; a warp may touch TMEM lanes 32·(warp%4) .. +31 =====
        const int q = warp & 3;
        const int c_first = ((warp - 2) >> 2) * EPI_WIDTH;  // this warp's share of the tile's columns
        int acc = 0;
        uint32_t acc_phase = 0;
        for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) {
            int b, tm, tn;
            grouped_tile_coords(tile, p.tiles_m, p.tiles_n, p.raster, b, tm, tn);
            if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag)) {
                if (lane == 0 && !*abort_flag) { *abort_flag = 1; atomicExch(p.status, GEMM_TIMEOUT_TMEM_FULL); }
                break;
            }
            tc_fence_after();
            drain_accumulator<T>(tmem_base + (uint32_t(q * 32) << 16) + acc * BN_ + c_first, EPI_WIDTH, C, p.c_staged != 0,
                                 epi_smem + (warp - 2) * EPI_WARP_BYTES, p.M, p.N, b, tm * BM + q * 32, tn * BN_ + c_first, lane);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(acc));
            if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1; }
        }
    }
    // Teardown: everyone meets, then the allocating warp frees TMEM.
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, Cfg::TMEM);
    }
}

// ---- the CTA-pair form: cta_group::2, one 256 × 256 tile per pair of SMs -------------------------
// Two CTAs of a cluster work on one tile.  CTA r of the pair owns rows r·128..r·128+127 of the
// tile (its own TMEM holds those accumulators) and loads, per 64-deep K block, its own 128 × 64
// slice of A and its own 64 × 128 half of the B panel: 32 KiB per stage instead of 48, so six
// stages fit, and every B element crosses L2 → shared memory once per pair instead of once per CTA.
// One thread of the leader CTA (rank 0) issues tcgen05.mma.cta_group::2 (M256 N256 K16): the
// tensor cores of both SMs read A from their own shared memory and the two B halves from both.
// Barrier protocol: the `full` barriers live in the leader (the peer's TMA loads complete on the
// leader's barrier through the .cta_group::2 form of the copy); `empty` and `tmem_full` exist in
// both CTAs and are signalled together by tcgen05.commit with a two-CTA mask; `tmem_empty` lives
// in the leader and collects the eight epilogue warps of both CTAs.  No multicast loads.
constexpr int P_STAGES = 6;
constexpr int P_B_STAGE_BYTES = B_BOX_BYTES * 2;                 // 64 K × 128 N
constexpr int P_STAGE_BYTES = A_STAGE_BYTES + P_B_STAGE_BYTES;   // 32 KiB
constexpr int P_SMEM_BYTES = P_STAGES * P_STAGE_BYTES + EPI_BYTES + 1024 + 256;
constexpr int PBM = 256;                                         // tile rows per pair

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Address of the same shared-memory location in CTA `rank` of this cluster.
__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t rank) {
    uint32_t out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(rank));
    return out;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap *map, uint32_t bar_cluster, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar_cluster), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives on the barrier at this shared-memory offset in every CTA of `mask` once all MMAs issued so far are done.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar, uint16_t mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(mask)
                 : "memory");
}
__host__ __device__ constexpr uint32_t make_idesc_pair(int ab_format) {
    return (1u << 4) | (uint32_t(ab_format) << 7) | (uint32_t(ab_format) << 10) | (0u << 15) | (1u << 16) |
           (uint32_t(BN >> 3) << 17) | (uint32_t(PBM >> 4) << 24);
}

struct PairParams {
    int M, N, K, batch;
    int tiles_m, tiles_n, num_tiles, k_blocks;  // tiles of 256 × 256
    int raster;   // rows of tiles per raster group
    int c_staged; // C takes 16-byte stores
    int *status;
};

template <typename T>
__global__ void __launch_bounds__(G_THREADS, 1)
    gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                             T *__restrict__ C, PairParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t epi_smem = smem_base + P_STAGES * P_STAGE_BYTES;
    constexpr int BAR_OFF = P_STAGES * P_STAGE_BYTES + EPI_BYTES;
    const uint32_t bars = smem_base + BAR_OFF;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (P_STAGES + s); };
    auto tfull_bar = [&](int a) { return bars + 8u * (2 * P_STAGES + a); };
    auto tempty_bar = [&](int a) { return bars + 8u * (2 * P_STAGES + ACC_STAGES + a); };
    constexpr int SLOT_OFF = 8 * (2 * P_STAGES + 2 * ACC_STAGES);
    const uint32_t tmem_slot = bars + SLOT_OFF;
    uint8_t *gen_base = smem_raw + (smem_base - smem_u32(smem_raw));
    volatile uint32_t *tmem_slot_ptr = reinterpret_cast<volatile uint32_t *>(gen_base + BAR_OFF + SLOT_OFF);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(gen_base + BAR_OFF + SLOT_OFF + 8);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();      // 0 = leader of the pair
    const int pair = blockIdx.x >> 1;             // cluster index (clusters are consecutive CTA pairs)
    const int num_pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < P_STAGES; ++s) {
            mbar_init(full_bar(s), 1);   // used in the leader only: its producer's arrive.expect_tx
            mbar_init(empty_bar(s), 1);  // one tcgen05.commit per use
        }
        for (int a = 0; a < ACC_STAGES; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 16);  // used in the leader only: 8 epilogue warps × 2 CTAs
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
    }
    if (warp == 1) tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // the peer's barriers exist before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_ptr;

    auto tile_coords = [&](int tile, int &b, int &tm, int &tn) { grouped_tile_coords(tile, p.tiles_m, p.tiles_n, p.raster, b, tm, tn); };

    if (warp == 0) {
        // ===== TMA producer (one per CTA; both complete on the LEADER's full barrier) =====
        if (lane == 0) {
            griddep_wait();  // the one thread that first touches global memory; every other role follows its loads
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = pair; tile < p.num_tiles && ok; tile += num_pairs) {
                int b, tm, tn;
                tile_coords(tile, b, tm, tn);
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1, abort_flag)) {
                        if (!*abort_flag) { *abort_flag = 1; atomicExch(p.status, GEMM_TIMEOUT_EMPTY); }
                        ok = false;
                        break;
                    }
                    const uint32_t sa = smem_base + stage * P_STAGE_BYTES;
                    const uint32_t sb = sa + A_STAGE_BYTES;
                    const uint32_t leader_full = mapa_u32(full_bar(stage), 0);
                    if (rank == 0) mbar_expect_tx(full_bar(stage), 2 * P_STAGE_BYTES);  // both CTAs' bytes
                    tma_load_3d_pair(sa, &tmap_a, leader_full, kb * BK, tm * PBM + int(rank) * BM, b);
#pragma unroll
                    for (int j = 0; j < 2; ++j)
                        tma_load_3d_pair(sb + j * B_BOX_BYTES, &tmap_b, leader_full, tn * BN + int(rank) * 128 + j * B_BOX_N, kb * BK, b);
                    if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
                }
            }
            if (*abort_flag) {
                const long long t0 = clock64();
                while (clock64() - t0 < 2000000ll) {}
            }
        }
    } else if (warp == 1) {
        // ===== MMA issuer: one thread of the leader CTA drives the tensor cores of both SMs =====
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = make_idesc_pair(std::is_same<T, bf16>::value ? 1 : 0);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int tile = pair; tile < p.num_tiles && ok; tile += num_pairs) {
                if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1, abort_flag)) {
                    if (!*abort_flag) { *abort_flag = 1; atomicExch(p.status, GEMM_TIMEOUT_TMEM_EMPTY); }
                    break;
                }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + acc * BN;
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
                        if (!*abort_flag) { *abort_flag = 1; atomicExch(p.status, GEMM_TIMEOUT_FULL); }
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sa = smem_base + stage * P_STAGE_BYTES;
                    const uint32_t sb = sa + A_STAGE_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint64_t adesc = make_smem_desc(sa + k * (UMMA_K * 2), 16, 1024);
                        const uint64_t bdesc = make_smem_desc(sb + k * (UMMA_K * 128), B_BOX_BYTES, 1024);
                        umma_f16_pair(tmem_d, adesc, bdesc, idesc, (kb | k) != 0);
                    }
                    umma_commit_pair(empty_bar(stage), 0x3);  // frees this stage in both CTAs
                    if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                umma_commit_pair(tfull_bar(acc), 0x3);  // accumulators of both CTAs complete
                if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1; }
            }
        }
    } else {
        // ===== epilogue: warps 2..9 of BOTH CTAs, each CTA drains its own 128 rows from its own TMEM;
        // two warps per TMEM lane quarter, each taking 128 of the 256 columns =====
        const int q = warp & 3;
        const int c_first = ((warp - 2) >> 2) * (BN / 2);
        int acc = 0;
        uint32_t acc_phase = 0;
        for (int tile = pair; tile < p.num_tiles; tile += num_pairs) {
            int b, tm, tn;
            tile_coords(tile, b, tm, tn);
            if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag)) {
                if (lane == 0 && !*abort_flag) { *abort_flag = 1; atomicExch(p.status, GEMM_TIMEOUT_TMEM_FULL); }
                break;
            }
            tc_fence_after();
            drain_accumulator<T>(tmem_base + (uint32_t(q * 32) << 16) + acc * BN + c_first, BN / 2, C, p.c_staged != 0,
                                 epi_smem + (warp - 2) * EPI_WARP_BYTES, p.M, p.N, b, tm * PBM + int(rank) * BM + q * 32,
                                 tn * BN + c_first, lane);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa_u32(tempty_bar(acc), 0));  // the leader's barrier collects all sixteen warps
            if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1; }
        }
    }
    // Teardown: neither CTA may leave (or free TMEM) while the other can still signal its barriers
    // or read its shared memory, so the whole pair meets first.
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

// ---- few rows of A (M <= 128): one row of tiles, split along K across a cluster ---------------------
// With at most one row of tiles the persistent kernels above put ceil(N/256) CTAs on 148 SMs and are
// bound by how fast so few SMs can pull B out of HBM.  Here a tile is 128 x 64 and the K range of a
// tile is divided among the CS <= 8 CTAs of a cluster: N/64 x CS CTAs, each streaming its own slab
// of B through a 6-stage TMA ring into tcgen05 MMAs (M128 N64 K16; rows beyond M are TMA zero fill
// and cost no HBM traffic).  Every CTA leaves its 128 x 64 fp32 partial in its own shared memory
// (over the drained ring); after a cluster barrier every CTA adds, for its share of the tile's columns,
// the partials of all ranks in rank order through distributed shared memory and writes those columns of
// the M live rows.  No workspace, no atomics: same bits every run.
constexpr int S_BN = 64;
constexpr int S_STAGES = 4;  // 96 KiB: two CTAs per SM
constexpr int S_STAGE_BYTES = A_STAGE_BYTES + B_BOX_BYTES;  // 16 KiB of A + 8 KiB of B
constexpr int S_PARTIAL_BYTES = BM * S_BN * 4;              // 32 KiB, reuses the ring after the main loop
constexpr int S_SMEM_BYTES = S_STAGES * S_STAGE_BYTES + 1024 + 256;
constexpr int S_TMEM_COLS = 64;
static_assert(S_PARTIAL_BYTES <= S_STAGES * S_STAGE_BYTES, "partial tile must fit in the ring");

struct SplitKParams {
    int M, N, K, batch;
    int tiles_n, k_blocks, kb_per_rank;
    int *status;
};

template <typename T>
__global__ void __launch_bounds__(NUM_THREADS, 1)
    gemm_tcgen05_splitk_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, T *__restrict__ C,
                               SplitKParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *gen_base = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bars = smem_base + S_STAGES * S_STAGE_BYTES;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (S_STAGES + s); };
    const uint32_t tfull_bar = bars + 8u * (2 * S_STAGES);
    constexpr int SLOT_OFF = 8 * (2 * S_STAGES + 1);
    const uint32_t tmem_slot = bars + SLOT_OFF;
    volatile uint32_t *tmem_slot_ptr = reinterpret_cast<volatile uint32_t *>(gen_base + S_STAGES * S_STAGE_BYTES + SLOT_OFF);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(gen_base + S_STAGES * S_STAGE_BYTES + SLOT_OFF + 8);
    float *partial = reinterpret_cast<float *>(gen_base);  // [BM][S_BN], valid after the main loop

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    uint32_t cs;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(cs));
    const uint32_t rank = cluster_ctarank();
    const int tn = blockIdx.x / cs;
    const int b = blockIdx.y;
    const int kb0 = int(rank) * p.kb_per_rank;
    const int kb1 = min(p.k_blocks, kb0 + p.kb_per_rank);
    const int nkb = max(kb1 - kb0, 0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < S_STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(tfull_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
    }
    if (warp == 1) tmem_alloc(tmem_slot, S_TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_ptr;

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            for (int kb = kb0; kb < kb1; ++kb) {
                if (!mbar_wait(empty_bar(stage), phase ^ 1, abort_flag)) {
                    if (!*abort_flag) { *abort_flag = 1; atomicExch(p.status, GEMM_TIMEOUT_EMPTY); }
                    break;
                }
                const uint32_t sa = smem_base + stage * S_STAGE_BYTES;
                mbar_expect_tx(full_bar(stage), S_STAGE_BYTES);
                tma_load_3d(sa, &tmap_a, full_bar(stage), kb * BK, 0, b);
                tma_load_3d(sa + A_STAGE_BYTES, &tmap_b, full_bar(stage), tn * S_BN, kb * BK, b);
                if (++stage == S_STAGES) { stage = 0; phase ^= 1; }
            }
            if (*abort_flag) {
                const long long t0 = clock64();
                while (clock64() - t0 < 2000000ll) {}
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && nkb > 0) {
            constexpr uint32_t idesc = make_idesc_n(std::is_same<T, bf16>::value ? 1 : 0, S_BN);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int kb = 0; kb < nkb; ++kb) {
                if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
                    if (!*abort_flag) { *abort_flag = 1; atomicExch(p.status, GEMM_TIMEOUT_FULL); }
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t sa = smem_base + stage * S_STAGE_BYTES;
                const uint32_t sb = sa + A_STAGE_BYTES;
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k) {
                    const uint64_t adesc = make_smem_desc(sa + k * (UMMA_K * 2), 16, 1024);
                    const uint64_t bdesc = make_smem_desc(sb + k * (UMMA_K * 128), B_BOX_BYTES, 1024);
                    umma_f16(tmem_base, adesc, bdesc, idesc, (kb | k) != 0);
                }
                umma_commit(empty_bar(stage));
                if (++stage == S_STAGES) { stage = 0; phase ^= 1; }
            }
            if (ok) umma_commit(tfull_bar);
        }
    } else {
        // epilogue warps: TMEM lane quarter warp % 4; only rows < M matter
        const int q = warp & 3;
        const int row = q * 32 + lane;
        bool have = false;
        uint32_t r0[32], r1[32];
        if (nkb > 0) {
            if (mbar_wait(tfull_bar, 0, abort_flag)) {
                tc_fence_after();
                tmem_ld_32x32b_x32(tmem_base + (uint32_t(q * 32) << 16) + 0, r0);
                tmem_ld_32x32b_x32(tmem_base + (uint32_t(q * 32) << 16) + 32, r1);
                tmem_ld_wait();
                have = true;
            } else if (lane == 0 && !*abort_flag) {
                *abort_flag = 1;
                atomicExch(p.status, GEMM_TIMEOUT_TMEM_FULL);
            }
        }
        // the ring is drained (every MMA that read it has completed): the partial tile goes on top of it
        // column-major [S_BN][BM]: the 32 lanes of a warp (32 rows) write neighbouring words
        if (row < p.M) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                partial[j * BM + row] = have ? __uint_as_float(r0[j]) : 0.f;
                partial[(32 + j) * BM + row] = have ? __uint_as_float(r1[j]) : 0.f;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // every CTA's partial is in place
    {
        // Reduce-scatter across the cluster: rank r sums columns [r, r+1) * S_BN / cs of the tile over all
        // ranks (always in rank order 0..cs-1, whoever does the adding) with 16-byte loads from the peers'
        // shared memory, and writes those columns of C.  Spreading the adds over the cluster matters:
        // 4-byte remote loads by one leader alone cost more than the whole main loop.
        const uint32_t pbase = smem_u32(partial);
        uint32_t peer[8];
#pragma unroll
        for (uint32_t r = 0; r < 8; ++r) peer[r] = r < cs ? mapa_u32(pbase, r) : 0u;
        const int cols_per = S_BN / int(cs);
        const int col0 = int(rank) * cols_per;
        const int quads = (p.M + 3) / 4;  // groups of four rows (rows are contiguous in the column-major partial)
        T *cbase = C + size_t(b) * p.M * p.N;
        for (int u = threadIdx.x; u < cols_per * quads; u += NUM_THREADS) {
            const int qd = u / cols_per, col = col0 + (u - qd * cols_per);  // neighbouring threads: neighbouring columns of C
            const uint32_t off = uint32_t(col * BM + qd * 4) * 4u;
            float4 v[8];
#pragma unroll
            for (uint32_t r = 0; r < 8; ++r) {
                if (r < cs) asm("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v[r].x), "=f"(v[r].y), "=f"(v[r].z), "=f"(v[r].w) : "r"(peer[r] + off));
                else v[r] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
            float4 acc = v[0];
#pragma unroll
            for (uint32_t r = 1; r < 8; ++r) { acc.x += v[r].x; acc.y += v[r].y; acc.z += v[r].z; acc.w += v[r].w; }
            const int gcol = tn * S_BN + col;
            if (gcol < p.N) {
                const float out4[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (qd * 4 + j < p.M) cbase[size_t(qd * 4 + j) * p.N + gcol] = from_compute<T>(out4[j]);
            }
        }
    }
    cluster_sync_all();  // nobody leaves while a peer may still read its shared memory
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, S_TMEM_COLS);
    }
}

// ---- a few rows of tiles (M of a few hundred): 256 x 256 pair tiles, K split across a cluster ---------
// What bounds a tile kernel on this part is how fast an SM can pull operands out of L2 (about 64 bytes
// per clock): a 128 x 256 tile of one CTA needs 96 bytes per clock to keep its tensor core busy, the
// 256 x 256 tile of a CTA pair needs 64 per SM because the B panel is shared.  A matrix with two or
// four rows of tiles gives too few pair tiles for the machine, so here the K range of one pair tile is
// divided among KS <= 4 pairs of one cluster (2·KS CTAs): every pair runs the cta_group::2 main loop
// over its slice of K; then CTA (slice s, half h) collects columns [s, s+1)·256/KS of rows h·128.. from
// all KS slices — each CTA pushes its fp32 partial of those columns into the collector's shared memory
// (over the drained ring) with remote stores — adds them in slice order and writes them to C.
// One tile per cluster, no workspace, no atomics: same bits every run.
constexpr int PS_PARTIAL_BYTES = BM * BN * 4;  // 128 KiB
constexpr int PS_SMEM_BYTES = P_STAGES * P_STAGE_BYTES + 1024 + 256;
static_assert(PS_PARTIAL_BYTES <= P_STAGES * P_STAGE_BYTES, "partial tile must fit in the ring");

struct PairSplitParams {
    int M, N, K, batch;
    int tiles_m, tiles_n, k_blocks, kb_per_slice;
    int *status;
};

template <typename T>
__global__ void __launch_bounds__(NUM_THREADS, 1)
    gemm_tcgen05_pair_splitk_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                                    T *__restrict__ C, PairSplitParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *gen_base = smem_raw + (smem_base - smem_u32(smem_raw));
    constexpr int BAR_OFF = P_STAGES * P_STAGE_BYTES;
    const uint32_t bars = smem_base + BAR_OFF;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (P_STAGES + s); };
    const uint32_t tfull_bar = bars + 8u * (2 * P_STAGES);
    constexpr int SLOT_OFF = 8 * (2 * P_STAGES + 1);
    const uint32_t tmem_slot = bars + SLOT_OFF;
    volatile uint32_t *tmem_slot_ptr = reinterpret_cast<volatile uint32_t *>(gen_base + BAR_OFF + SLOT_OFF);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(gen_base + BAR_OFF + SLOT_OFF + 8);
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    uint32_t csize;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(csize));
    const uint32_t rank = cluster_ctarank();
    const uint32_t half = rank & 1u;        // which 128 rows of the pair tile
    const uint32_t slice = rank >> 1;       // which part of K
    const uint32_t leader = rank & ~1u;     // the CTA of this pair that issues the MMAs
    const uint32_t ks = csize >> 1;
    const int tile = blockIdx.x / csize;
    const int per_batch = p.tiles_m * p.tiles_n;
    const int b = tile / per_batch;
    const int tm = (tile - b * per_batch) / p.tiles_n;
    const int tn = tile - b * per_batch - tm * p.tiles_n;
    const int kb0 = int(slice) * p.kb_per_slice;
    const int kb1 = min(p.k_blocks, kb0 + p.kb_per_slice);
    const int nkb = max(kb1 - kb0, 0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < P_STAGES; ++s) {
            mbar_init(full_bar(s), 1);   // used in the pair's leader only
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(tfull_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
    }
    if (warp == 1) tmem_alloc_pair(tmem_slot, BN);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // the peer's barriers exist before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_ptr;

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            for (int kb = kb0; kb < kb1; ++kb) {
                if (!mbar_wait(empty_bar(stage), phase ^ 1, abort_flag)) {
                    if (!*abort_flag) { *abort_flag = 1; atomicExch(p.status, GEMM_TIMEOUT_EMPTY); }
                    break;
                }
                const uint32_t sa = smem_base + stage * P_STAGE_BYTES;
                const uint32_t sb = sa + A_STAGE_BYTES;
                const uint32_t leader_full = mapa_u32(full_bar(stage), leader);
                if (half == 0) mbar_expect_tx(full_bar(stage), 2 * P_STAGE_BYTES);  // both CTAs' bytes
                tma_load_3d_pair(sa, &tmap_a, leader_full, kb * BK, tm * PBM + int(half) * BM, b);
#pragma unroll
                for (int j = 0; j < 2; ++j)
                    tma_load_3d_pair(sb + j * B_BOX_BYTES, &tmap_b, leader_full, tn * BN + int(half) * 128 + j * B_BOX_N, kb * BK, b);
                if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
            }
            if (*abort_flag) {
                const long long t0 = clock64();
                while (clock64() - t0 < 2000000ll) {}
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && half == 0 && nkb > 0) {
            constexpr uint32_t idesc = make_idesc_pair(std::is_same<T, bf16>::value ? 1 : 0);
            const uint16_t mask = uint16_t(0x3u << leader);  // this pair's two CTAs
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int kb = 0; kb < nkb; ++kb) {
                if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
                    if (!*abort_flag) { *abort_flag = 1; atomicExch(p.status, GEMM_TIMEOUT_FULL); }
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t sa = smem_base + stage * P_STAGE_BYTES;
                const uint32_t sb = sa + A_STAGE_BYTES;
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k) {
                    const uint64_t adesc = make_smem_desc(sa + k * (UMMA_K * 2), 16, 1024);
                    const uint64_t bdesc = make_smem_desc(sb + k * (UMMA_K * 128), B_BOX_BYTES, 1024);
                    umma_f16_pair(tmem_base, adesc, bdesc, idesc, (kb | k) != 0);
                }
                umma_commit_pair(empty_bar(stage), mask);
                if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
            }
            if (ok) umma_commit_pair(tfull_bar, mask);  // both CTAs' accumulators complete
        }
    }
    // ---- combine the KS partial tiles ----
    // Barrier 1: every CTA of the cluster has finished its main loop (its epilogue warps arrive only after
    // their accumulator is complete), so every ring is drained and may be overwritten.
    bool have = false;
    if (warp >= 2 && nkb > 0) {
        if (mbar_wait(tfull_bar, 0, abort_flag)) {
            tc_fence_after();
            have = true;
        } else if (lane == 0 && !*abort_flag) {
            *abort_flag = 1;
            atomicExch(p.status, GEMM_TIMEOUT_TMEM_FULL);
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    // Push: slice o of the cluster owns columns [o, o+1)·256/KS.  Each epilogue warp sends its 32 rows of
    // every 32-column chunk to the owner's receive buffer for this slice — remote 16-byte stores, which
    // unlike remote loads nobody has to wait for.  A receive buffer is row-major [128][256/KS] floats with
    // the 16-byte chunks of a row XOR-swizzled by the row number (conflict-free for writer and reader).
    const int cols_per = BN / int(ks);
    const uint32_t pitch = uint32_t(cols_per) * 4u;
    const uint32_t recv_bytes = uint32_t(BM) * pitch;  // per source slice; KS of them = 128 KiB
    if (warp >= 2) {
        tc_fence_after();
        const int q = warp & 3;
        const int row = q * 32 + lane;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
            uint32_t r[32];
            if (have) {
                tmem_ld_32x32b_x32(tmem_base + (uint32_t(q * 32) << 16) + c0, r);
                tmem_ld_wait();
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) r[j] = 0u;
            }
            const int owner = c0 / cols_per;
            const int cin = c0 - owner * cols_per;  // first column inside the owner's share
            const uint32_t dst = mapa_u32(smem_base + slice * recv_bytes + uint32_t(row) * pitch, uint32_t(2 * owner) + half);
#pragma unroll
            for (int v = 0; v < 8; ++v) {
                const uint32_t chunk = uint32_t(cin / 4 + v) ^ uint32_t(row & 7);
                asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst + chunk * 16u), "r"(r[4 * v + 0]),
                             "r"(r[4 * v + 1]), "r"(r[4 * v + 2]), "r"(r[4 * v + 3])
                             : "memory");
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // barrier 2: every slice's share has arrived (release/acquire over the cluster)
    {
        // Local sum over the KS receive buffers in slice order, round once, 8-byte stores: a warp covers
        // 128 consecutive columns of one row of C.
        const int chunks_per_row = cols_per / 4;
        const int row_base = tm * PBM + int(half) * BM;
        const int live = min(BM, p.M - row_base);  // rows of this CTA inside C (may be <= 0)
        const int col_base = tn * BN + int(slice) * cols_per;
        T *cbase = C + size_t(b) * p.M * p.N;
        const bool vec_ok = (reinterpret_cast<uintptr_t>(C) & 7) == 0;  // N % 8 == 0 on this path
        for (int u = threadIdx.x; u < max(live, 0) * chunks_per_row; u += NUM_THREADS) {
            const int row = u / chunks_per_row, chunk = u - row * chunks_per_row;
            const uint32_t off = uint32_t(row) * pitch + ((uint32_t(chunk) ^ uint32_t(row & 7)) << 4);
            float4 acc = *reinterpret_cast<const float4 *>(gen_base + off);
            for (uint32_t s = 1; s < ks; ++s) {
                const float4 v = *reinterpret_cast<const float4 *>(gen_base + s * recv_bytes + off);
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
            }
            const int gcol = col_base + chunk * 4;
            T *dst = cbase + size_t(row_base + row) * p.N + gcol;
            if (vec_ok && gcol + 4 <= p.N) {
                uint2 o;
                o.x = pack2<T>(acc.x, acc.y);
                o.y = pack2<T>(acc.z, acc.w);
                *reinterpret_cast<uint2 *>(dst) = o;
            } else {
                const float out4[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (gcol + j < p.N) dst[j] = from_compute<T>(out4[j]);
            }
        }
    }
    // the pair frees its TMEM together
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, BN);
    }
}

// ---- a few rows of tiles, K split over INDEPENDENT pairs through a workspace ----------------------------
// The cluster form above pays two cluster barriers, a late start (clusters of 4–8 CTAs must find room in one GPC)
// and the exchange of partials, about 8 µs, so it only helps when K is long.  Here every (tile, K slice) is an
// ordinary CTA pair of its own, launched cooperatively so that all of them are resident: the pair runs the
// cta_group::2 main loop over its slice, and then the KS pairs of a tile share out the finishing — pair s finishes
// the s-th share of the tile's 32-column blocks.  A CTA writes the blocks that OTHER pairs finish to the caller's
// workspace in the order the values come out of TMEM (every store instruction of a warp covers 512 contiguous
// bytes), counts itself in on a per-(tile, half) counter, waits (bounded) until all KS have, then adds, for its
// own blocks, the partials in slice order — its own straight from TMEM, the others out of L2 — rounds once and
// writes C.  What bounds this phase is what one SM can push into and pull out of L2 (about 32 and 64 bytes per
// clock, measured); sharing it out means a CTA moves (KS-1)/KS of a 128 KiB partial each way instead of one CTA
// pulling KS-1 whole partials.  The sum has the same order whoever runs first, so the same bits.  No atomics on
// data.  Workspace: tiles × KS × 256 × 256 floats.
struct PairWsParams {
    int M, N, K, batch;
    int tiles_m, tiles_n, k_blocks, kb_per_slice, ks;
    int c_staged;
    int *status;
    float *partial;          // [tile][slice][half][128 rows × 256 columns in TMEM order]
    unsigned long long *counters;  // [tile][half]: grows by WSK_STEP per launch
};
constexpr int W_THREADS = 256;          // eight warps; warps 0 and 1 feed the main loop first, then all eight store and finish
constexpr int WS_HALF_FLOATS = BM * BN;  // 32768 floats = 128 KiB per CTA and slice
constexpr int GEMM_TIMEOUT_SLICES = 7;
constexpr unsigned int WSK_STEP = 840;  // divisible by every KS up to 8
constexpr int WSK_BANKS = 8;             // one set of counters per stream that launches this kernel
__device__ unsigned long long g_wsk_counters[WSK_BANKS][512];

__device__ __forceinline__ unsigned long long ld_acquire_gpu(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_add(unsigned long long *p, unsigned long long v) {
    asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// A warp's block of 32 rows × 32 columns, one row per lane in r[32] as fp32 bit patterns, rounded once and written
// to C: turned round in 2 KiB of shared memory (rows of 64 bytes, their 16-byte chunks XOR-swizzled by half the row
// number: no bank conflicts either way) and stored with four lanes per row when `staged`, else row by row.
template <typename T>
__device__ __forceinline__ void emit_chunk32(const uint32_t (&r)[32], T *C, bool staged, uint32_t stage_smem, int M, int N, int b, int row0,
                                             int col, int lane) {
    if (row0 >= M || col >= N) return;
    if (staged) {
        const uint32_t mine = stage_smem + lane * 64;
        const int sw = (lane >> 1) & 3;
#pragma unroll
        for (int v = 0; v < 4; ++v)
            st_shared_v4(mine + ((v ^ sw) << 4),
                         pack2<T>(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1])),
                         pack2<T>(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3])),
                         pack2<T>(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5])),
                         pack2<T>(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7])));
        __syncwarp();
        const int chunk = lane & 3;
        const int gcol = col + chunk * 8;
        uint4 v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int rr = i * 8 + (lane >> 2);
            v[i] = ld_shared_v4(stage_smem + rr * 64 + ((chunk ^ ((rr >> 1) & 3)) << 4));
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int rr = i * 8 + (lane >> 2);
            if (row0 + rr < M && gcol < N) *reinterpret_cast<uint4 *>(C + (size_t(b) * M + row0 + rr) * N + gcol) = v[i];
        }
        __syncwarp();
    } else if (row0 + lane < M) {
        T *crow = C + (size_t(b) * M + row0 + lane) * N;
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (col + j < N) crow[col + j] = from_compute<T>(__uint_as_float(r[j]));
    }
}

template <typename T>
__global__ void __launch_bounds__(W_THREADS, 1)
    gemm_tcgen05_pair_wsk_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                                 T *__restrict__ C, PairWsParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *gen_base = smem_raw + (smem_base - smem_u32(smem_raw));
    constexpr int BAR_OFF = P_STAGES * P_STAGE_BYTES;
    const uint32_t bars = smem_base + BAR_OFF;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (P_STAGES + s); };
    const uint32_t tfull_bar = bars + 8u * (2 * P_STAGES);
    constexpr int SLOT_OFF = 8 * (2 * P_STAGES + 1);
    const uint32_t tmem_slot = bars + SLOT_OFF;
    volatile uint32_t *tmem_slot_ptr = reinterpret_cast<volatile uint32_t *>(gen_base + BAR_OFF + SLOT_OFF);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(gen_base + BAR_OFF + SLOT_OFF + 8);
    volatile int *go_flag = reinterpret_cast<volatile int *>(gen_base + BAR_OFF + SLOT_OFF + 12);
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t half = cluster_ctarank();  // which 128 rows of the pair tile; rank 0 issues the MMAs
    const int unit = blockIdx.x >> 1;         // (tile, slice)
    const int tile = unit / p.ks;
    const int slice = unit - tile * p.ks;
    const int per_batch = p.tiles_m * p.tiles_n;
    const int b = tile / per_batch;
    const int tm = (tile - b * per_batch) / p.tiles_n;
    const int tn = tile - b * per_batch - tm * p.tiles_n;
    const int kb0 = slice * p.kb_per_slice;
    const int kb1 = min(p.k_blocks, kb0 + p.kb_per_slice);
    const int nkb = max(kb1 - kb0, 0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < P_STAGES; ++s) {
            mbar_init(full_bar(s), 1);   // used in the leader only
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(tfull_bar, 1);
        *abort_flag = 0;
        *go_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
    }
    if (warp == 1) tmem_alloc_pair(tmem_slot, BN);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // the peer's barriers exist before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_ptr;
    // The counter of this (tile, half) only ever grows, by WSK_STEP per launch whatever KS is.  Read before this
    // CTA has counted itself in, it lies in [base, base + WSK_STEP) with base the value the last launch left, so the
    // value to wait for is known now and the count-in itself needs no answer from L2.
    unsigned long long *arrived = p.counters + tile * 2 + half;
    unsigned long long target = 0;
    if (threadIdx.x == 0) target = (ld_acquire_gpu(arrived) / WSK_STEP + 1ull) * WSK_STEP;
    bool have = false;  // this CTA's accumulator is complete

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            for (int kb = kb0; kb < kb1; ++kb) {
                if (!mbar_wait(empty_bar(stage), phase ^ 1, abort_flag)) {
                    if (!*abort_flag) { *abort_flag = 1; atomicExch(p.status, GEMM_TIMEOUT_EMPTY); }
                    break;
                }
                const uint32_t sa = smem_base + stage * P_STAGE_BYTES;
                const uint32_t sb = sa + A_STAGE_BYTES;
                const uint32_t leader_full = mapa_u32(full_bar(stage), 0);
                if (half == 0) mbar_expect_tx(full_bar(stage), 2 * P_STAGE_BYTES);  // both CTAs' bytes
                tma_load_3d_pair(sa, &tmap_a, leader_full, kb * BK, tm * PBM + int(half) * BM, b);
#pragma unroll
                for (int j = 0; j < 2; ++j)
                    tma_load_3d_pair(sb + j * B_BOX_BYTES, &tmap_b, leader_full, tn * BN + int(half) * 128 + j * B_BOX_N, kb * BK, b);
                if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
            }
            if (*abort_flag) {
                const long long t0 = clock64();
                while (clock64() - t0 < 2000000ll) {}
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && half == 0 && nkb > 0) {
            constexpr uint32_t idesc = make_idesc_pair(std::is_same<T, bf16>::value ? 1 : 0);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int kb = 0; kb < nkb; ++kb) {
                if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
                    if (!*abort_flag) { *abort_flag = 1; atomicExch(p.status, GEMM_TIMEOUT_FULL); }
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t sa = smem_base + stage * P_STAGE_BYTES;
                const uint32_t sb = sa + A_STAGE_BYTES;
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k) {
                    const uint64_t adesc = make_smem_desc(sa + k * (UMMA_K * 2), 16, 1024);
                    const uint64_t bdesc = make_smem_desc(sb + k * (UMMA_K * 128), B_BOX_BYTES, 1024);
                    umma_f16_pair(tmem_base, adesc, bdesc, idesc, (kb | k) != 0);
                }
                umma_commit_pair(empty_bar(stage), 0x3);
                if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
            }
            if (ok) umma_commit_pair(tfull_bar, 0x3);  // both CTAs' accumulators complete
        }
    }
    __syncwarp();  // lane 0 of warps 0 and 1 is back from its loop: all eight warps take part from here on
    if (nkb > 0) {
        if (mbar_wait(tfull_bar, 0, abort_flag)) {
            tc_fence_after();
            have = true;
        } else if (lane == 0 && !*abort_flag) {
            *abort_flag = 1;
            atomicExch(p.status, GEMM_TIMEOUT_TMEM_FULL);
        }
    }
    // two warps per TMEM lane quarter; they take the 32-column blocks of a list in turn
    const int q = warp & 3, wh = warp >> 2;
    const uint32_t tmem_row = tmem_base + (uint32_t(q * 32) << 16);
    const int my_c0 = (8 * slice) / p.ks, my_c1 = (8 * (slice + 1)) / p.ks;  // the blocks this pair finishes (KS <= 8: at least one)
    {
        // ---- the blocks other pairs finish: TMEM → this slice's place in the workspace ----
        float4 *mine = reinterpret_cast<float4 *>(p.partial + ((size_t(tile) * p.ks + slice) * 2 + half) * WS_HALF_FLOATS);
        int n = 0;
#pragma unroll 1
        for (int c = 0; c < 8; ++c) {
            if (c >= my_c0 && c < my_c1) continue;
            if ((n++ & 1) != wh) continue;
            uint32_t r[32];
            if (have) {
                tmem_ld_32x32b_x32(tmem_row + c * 32, r);
                tmem_ld_wait();
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) r[j] = 0u;
            }
#pragma unroll
            for (int v = 0; v < 8; ++v)
                mine[((q * 8 + c) * 8 + v) * 32 + lane] =
                    make_float4(__uint_as_float(r[4 * v + 0]), __uint_as_float(r[4 * v + 1]), __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) {
        // The barrier orders every warp's stores before this release, and a release is cumulative: they are visible
        // device-wide before the count.  All KS pairs of the tile are resident (a cooperative launch) and none waits
        // before it has counted itself in, so the wait ends; it is bounded all the same.
        red_release_add(arrived, WSK_STEP / unsigned(p.ks));
        const long long t0 = clock64();
        bool ok = true;
        while (ld_acquire_gpu(arrived) < target) {
            if (clock64() - t0 > WAIT_LIMIT_CYCLES) { ok = false; break; }
        }
        if (!ok) atomicExch(p.status, GEMM_TIMEOUT_SLICES);
        *go_flag = ok ? 1 : 0;
    }
    __syncthreads();
    if (*go_flag) {
        // ---- this pair's own blocks: partials in slice order, rounded once, written to C ----
        tc_fence_after();
        const uint32_t stage_smem = smem_base + warp * EPI_WARP_BYTES;  // the ring is drained: reuse it for turning the blocks
        const float4 *base = reinterpret_cast<const float4 *>(p.partial + (size_t(tile) * p.ks * 2 + half) * WS_HALF_FLOATS);
        const size_t slice_stride = size_t(2) * WS_HALF_FLOATS / 4;  // float4s between consecutive slices of this half
        const int row0 = tm * PBM + int(half) * BM + q * 32;
        // A batch = the 8 float4 a thread needs of one of its blocks from one other slice.  Up to four batches are
        // requested before the first is added, so the trip to L2 (some 2000 cycles with every SM storing and loading
        // at once) is paid once per four, not once each; the adding keeps slice order, this pair's own slice coming
        // straight from TMEM at its place in that order.
        const int others = p.ks - 1;
        const int my_blocks = (my_c1 - my_c0 - wh + 1) >> 1;  // blocks my_c0 + wh, + 2, ...
        const int batches = my_blocks * others;
        constexpr int NB = 4;
        float4 acc[8];
        bool started = false, own_done = false;
        auto fold = [&](const float4(&x)[8]) {
#pragma unroll
            for (int v = 0; v < 8; ++v) {
                if (!started) acc[v] = x[v];
                else { acc[v].x += x[v].x; acc[v].y += x[v].y; acc[v].z += x[v].z; acc[v].w += x[v].w; }
            }
            started = true;
        };
        auto fold_own = [&](int c) {
            uint32_t u[32];
            if (have) {
                tmem_ld_32x32b_x32(tmem_row + c * 32, u);
                tmem_ld_wait();
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) u[j] = 0u;
            }
            float4 x[8];
#pragma unroll
            for (int v = 0; v < 8; ++v)
                x[v] = make_float4(__uint_as_float(u[4 * v + 0]), __uint_as_float(u[4 * v + 1]), __uint_as_float(u[4 * v + 2]), __uint_as_float(u[4 * v + 3]));
            fold(x);
            own_done = true;
        };
#pragma unroll 1
        for (int j0 = 0; j0 < batches; j0 += NB) {
            float4 t[NB][8];
#pragma unroll
            for (int s = 0; s < NB; ++s) {
                const int j = j0 + s;
                if (j < batches) {
                    const int bi = j / others, oi = j - bi * others;
                    const int sl = oi + (oi >= slice ? 1 : 0), c = my_c0 + wh + 2 * bi;
                    const float4 *src = base + sl * slice_stride + size_t(((q * 8 + c) * 8) * 32 + lane);
#pragma unroll
                    for (int v = 0; v < 8; ++v) t[s][v] = __ldcg(src + v * 32);
                }
            }
#pragma unroll
            for (int s = 0; s < NB; ++s) {
                const int j = j0 + s;
                if (j < batches) {
                    const int bi = j / others, oi = j - bi * others;
                    const int sl = oi + (oi >= slice ? 1 : 0), c = my_c0 + wh + 2 * bi;
                    if (oi == 0) { started = false; own_done = false; }
                    if (!own_done && slice < sl) fold_own(c);
                    fold(t[s]);
                    if (oi == others - 1) {
                        if (!own_done) fold_own(c);
                        uint32_t r[32];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            r[4 * i + 0] = __float_as_uint(acc[i].x);
                            r[4 * i + 1] = __float_as_uint(acc[i].y);
                            r[4 * i + 2] = __float_as_uint(acc[i].z);
                            r[4 * i + 3] = __float_as_uint(acc[i].w);
                        }
                        emit_chunk32<T>(r, C, p.c_staged != 0, stage_smem, p.M, p.N, b, row0, tn * BN + c * 32, lane);
                    }
                }
            }
        }
    }
    // the pair frees its TMEM together
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, BN);
    }
}

// ---- float32 on the tensor cores: three TF32 products per fp32 product ------------------------------
// kind::tf32 reads 32-bit words and keeps 10 mantissa bits, which alone misses the 1e-5 bound.  Each
// operand is therefore split IN SHARED MEMORY into hi = round-to-tf32(x) and lo = x − hi (exact in
// fp32, |lo| ≤ 2^-11 |x|), and the kernel accumulates  Ahi·Bhi + Alo·Bhi + Ahi·Blo  in fp32 TMEM.
// What is dropped (Alo·Blo, and the tf32 truncation of lo) is ~2^-21 relative to |a||b|.
//   warp 0      TMA producer: raw fp32 tiles (A 128×32, B 32×128 as four 32-column panels)
//   warps 6-9   splitters: rewrite the raw tile as hi in place, write lo beside it, fence to the
//               async proxy, signal the MMA warp
//   warp 1      MMA issuer: 4 K-steps × 3 products of tcgen05.mma.kind::tf32 (M128 N128 K8) per stage
//   warps 2-5   epilogue: TMEM → fp32 → 16-byte stores
// The caller passes no workspace: nothing is pre-split in global memory.
constexpr int F_BN = 128, F_BK = 32, F_UMMA_K = 8;
constexpr int F_STAGES = 3;
constexpr int F_A_BYTES = BM * F_BK * 4;                 // 16 KiB
constexpr int F_B_BOX_N = 32;                            // 32 fp32 = one 128-byte swizzle row
constexpr int F_B_BOX_BYTES = F_BK * F_B_BOX_N * 4;      // 4 KiB
constexpr int F_B_BYTES = F_B_BOX_BYTES * (F_BN / F_B_BOX_N);  // 16 KiB
constexpr int F_RAW_BYTES = F_A_BYTES + F_B_BYTES;       // what TMA delivers per stage
constexpr int F_STAGE_BYTES = 2 * F_RAW_BYTES;           // hi + lo of both operands: 64 KiB
constexpr int F_SMEM_BYTES = F_STAGES * F_STAGE_BYTES + 1024 + 256;
constexpr int F_TMEM_COLS = ACC_STAGES * F_BN;           // 256
constexpr int F_THREADS = 320;
enum { GEMM_TIMEOUT_RAW = 5, GEMM_TIMEOUT_SPLIT = 6 };

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ float round_tf32(float x) {
    uint32_t u;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
    return __uint_as_float(u);
}
// D f32 (1<<4), A and B tf32 (format 2), A K-major, B MN-major, N = 128, M = 128
__host__ __device__ constexpr uint32_t make_idesc_tf32() {
    return (1u << 4) | (2u << 7) | (2u << 10) | (0u << 15) | (1u << 16) | (uint32_t(F_BN >> 3) << 17) | (uint32_t(BM >> 4) << 24);
}

__global__ void __launch_bounds__(F_THREADS, 1)
    gemm_tf32x3_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, float *__restrict__ C,
                       GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *gen_base = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bars = smem_base + F_STAGES * F_STAGE_BYTES;
    auto raw_bar = [&](int s) { return bars + 8u * s; };                       // TMA → splitters
    auto split_bar = [&](int s) { return bars + 8u * (F_STAGES + s); };        // splitters → MMA
    auto empty_bar = [&](int s) { return bars + 8u * (2 * F_STAGES + s); };    // MMA → TMA
    auto tfull_bar = [&](int a) { return bars + 8u * (3 * F_STAGES + a); };
    auto tempty_bar = [&](int a) { return bars + 8u * (3 * F_STAGES + ACC_STAGES + a); };
    constexpr int SLOT_OFF = 8 * (3 * F_STAGES + 2 * ACC_STAGES);
    const uint32_t tmem_slot = bars + SLOT_OFF;
    volatile uint32_t *tmem_slot_ptr = reinterpret_cast<volatile uint32_t *>(gen_base + F_STAGES * F_STAGE_BYTES + SLOT_OFF);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(gen_base + F_STAGES * F_STAGE_BYTES + SLOT_OFF + 8);
    // stage layout: [A hi | B hi | A lo | B lo]; TMA fills the first two, which the splitters round in place
    auto a_hi = [&](int s) { return smem_base + s * F_STAGE_BYTES; };
    auto b_hi = [&](int s) { return smem_base + s * F_STAGE_BYTES + F_A_BYTES; };
    auto a_lo = [&](int s) { return smem_base + s * F_STAGE_BYTES + F_RAW_BYTES; };
    auto b_lo = [&](int s) { return smem_base + s * F_STAGE_BYTES + F_RAW_BYTES + F_A_BYTES; };

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < F_STAGES; ++s) {
            mbar_init(raw_bar(s), 1);
            mbar_init(split_bar(s), 4);  // one arrival per splitter warp
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < ACC_STAGES; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 4);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
    }
    if (warp == 1) tmem_alloc(tmem_slot, F_TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_ptr;

    auto tile_coords = [&](int tile, int &b, int &tm, int &tn) { grouped_tile_coords(tile, p.tiles_m, p.tiles_n, p.raster, b, tm, tn); };
    if (warp == 0) {
        // ===== TMA producer =====
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
                int b, tm, tn;
                tile_coords(tile, b, tm, tn);
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1, abort_flag)) {
                        if (!*abort_flag) { *abort_flag = 1; atomicExch(p.status, GEMM_TIMEOUT_EMPTY); }
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(raw_bar(stage), F_RAW_BYTES);
                    tma_load_3d(a_hi(stage), &tmap_a, raw_bar(stage), kb * F_BK, tm * BM, b);
#pragma unroll
                    for (int j = 0; j < F_BN / F_B_BOX_N; ++j)
                        tma_load_3d(b_hi(stage) + j * F_B_BOX_BYTES, &tmap_b, raw_bar(stage), tn * F_BN + j * F_B_BOX_N, kb * F_BK, b);
                    if (++stage == F_STAGES) { stage = 0; phase ^= 1; }
                }
            }
            if (*abort_flag) {
                const long long t0 = clock64();
                while (clock64() - t0 < 2000000ll) {}
            }
        }
    } else if (warp == 1) {
        // ===== MMA issuer =====
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_tf32();
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
                if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1, abort_flag)) {
                    if (!*abort_flag) { *abort_flag = 1; atomicExch(p.status, GEMM_TIMEOUT_TMEM_EMPTY); }
                    break;
                }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + acc * F_BN;
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    if (!mbar_wait(split_bar(stage), phase, abort_flag)) {
                        if (!*abort_flag) { *abort_flag = 1; atomicExch(p.status, GEMM_TIMEOUT_SPLIT); }
                        ok = false;
                        break;
                    }
                    tc_fence_after();
#pragma unroll
                    for (int k = 0; k < F_BK / F_UMMA_K; ++k) {
                        // A: K-major; 8 fp32 = 32 bytes per K step inside the 128-byte swizzle row
                        const uint64_t ah = make_smem_desc(a_hi(stage) + k * 32, 16, 1024);
                        const uint64_t al = make_smem_desc(a_lo(stage) + k * 32, 16, 1024);
                        // B: N-major. 32-bit N-major operands exist only in the 128-byte swizzle of
                        // 32-byte chunks (mode 1): its atom is 32 columns x 4 K rows = 512 bytes, so one
                        // K = 8 step spans two atoms 512 bytes apart; 32-column panels are 4096 bytes apart.
                        const uint64_t bh = make_smem_desc(b_hi(stage) + k * 1024, F_B_BOX_BYTES, 512, 1);
                        const uint64_t bl = make_smem_desc(b_lo(stage) + k * 1024, F_B_BOX_BYTES, 512, 1);
                        umma_tf32(tmem_d, al, bh, idesc, (kb | k) != 0);  // small terms first
                        umma_tf32(tmem_d, ah, bl, idesc, 1);
                        umma_tf32(tmem_d, ah, bh, idesc, 1);
                    }
                    umma_commit(empty_bar(stage));
                    if (++stage == F_STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                umma_commit(tfull_bar(acc));
                if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1; }
            }
        }
    } else if (warp < 6) {
        // ===== epilogue: warps 2..5 → TMEM lane quarter warp % 4 =====
        const int q = warp & 3;
        int acc = 0;
        uint32_t acc_phase = 0;
        const bool vec_ok = (p.N % 4) == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0;
        for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) {
            int b, tm, tn;
            tile_coords(tile, b, tm, tn);
            if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag)) {
                if (lane == 0 && !*abort_flag) { *abort_flag = 1; atomicExch(p.status, GEMM_TIMEOUT_TMEM_FULL); }
                break;
            }
            tc_fence_after();
            const int row = tm * BM + q * 32 + lane;
            float *crow = C + (size_t(b) * p.M + row) * p.N;
#pragma unroll 1
            for (int c0 = 0; c0 < F_BN; c0 += 32) {
                uint32_t r[32];
                tmem_ld_32x32b_x32(tmem_base + (uint32_t(q * 32) << 16) + acc * F_BN + c0, r);
                tmem_ld_wait();
                const int col = tn * F_BN + c0;
                if (row < p.M) {
                    if (vec_ok && col + 32 <= p.N) {
#pragma unroll
                        for (int v = 0; v < 8; ++v)
                            *reinterpret_cast<uint4 *>(crow + col + 4 * v) = make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (col + j < p.N) crow[col + j] = __uint_as_float(r[j]);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(acc));
            if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1; }
        }
    } else {
        // ===== splitters: warps 6..9, 128 threads; 2048 float4 per stage (A and B raw tiles) =====
        const int t = threadIdx.x - 6 * 32;
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
            for (int kb = 0; kb < p.k_blocks; ++kb) {
                if (!mbar_wait(raw_bar(stage), phase, abort_flag)) {
                    if (lane == 0 && !*abort_flag) { *abort_flag = 1; atomicExch(p.status, GEMM_TIMEOUT_RAW); }
                    ok = false;
                    break;
                }
                float4 *hi = reinterpret_cast<float4 *>(gen_base + stage * F_STAGE_BYTES);
                float4 *lo = reinterpret_cast<float4 *>(gen_base + stage * F_STAGE_BYTES + F_RAW_BYTES);
#pragma unroll 4
                for (int i = t; i < F_RAW_BYTES / 16; i += 128) {
                    const float4 x = hi[i];
                    float4 h, l;
                    h.x = round_tf32(x.x); l.x = x.x - h.x;
                    h.y = round_tf32(x.y); l.y = x.y - h.y;
                    h.z = round_tf32(x.z); l.z = x.z - h.z;
                    h.w = round_tf32(x.w); l.w = x.w - h.w;
                    hi[i] = h;
                    lo[i] = l;
                }
                fence_proxy_async_smem();  // these generic-proxy writes are read next by the tensor core
                __syncwarp();
                if (lane == 0) mbar_arrive(split_bar(stage));
                if (++stage == F_STAGES) { stage = 0; phase ^= 1; }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, F_TMEM_COLS);
    }
}

// ---- float32, CTA-pair form: a 256 × 256 tile per pair of SMs ---------------------------------------
// The one-CTA kernel above is bound by shared-memory bandwidth, not by the tensor pipe: per
// 128 × 128 × 32 block the splitters move 96 KiB and the three MMAs read 96 KiB of operands.  With
// cta_group::2 each CTA still loads and splits a 128 × 32 slice of A and a 32 × 128 half of B
// (same 64 KiB stage, same splitter work) but the pair computes 256 × 256, so every operand byte
// read from shared memory feeds twice the flops.  Protocol as in the bf16 pair kernel, plus the
// split step: each CTA's TMA completes on its OWN `raw` barrier (its own splitters wait there);
// all eight splitter warps of the pair arrive on the LEADER's `split` barrier (release at cluster
// scope, after the proxy fence), where the one MMA thread waits with a cluster-scope acquire.
constexpr int FP_BN = 256;
constexpr int FP_TMEM_COLS = ACC_STAGES * FP_BN;  // 512

__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
        if (mbar_try_wait_cluster(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > WAIT_LIMIT_CYCLES) return false;
    }
}
__device__ __forceinline__ void umma_tf32_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D f32, A and B tf32, A K-major, B MN-major, N = 256, M = 256 (128 rows in each CTA's TMEM)
__host__ __device__ constexpr uint32_t make_idesc_tf32_pair() {
    return (1u << 4) | (2u << 7) | (2u << 10) | (0u << 15) | (1u << 16) | (uint32_t(FP_BN >> 3) << 17) | (uint32_t(PBM >> 4) << 24);
}

__global__ void __launch_bounds__(F_THREADS, 1)
    gemm_tf32x3_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                            float *__restrict__ C, PairParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *gen_base = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bars = smem_base + F_STAGES * F_STAGE_BYTES;
    auto raw_bar = [&](int s) { return bars + 8u * s; };                       // this CTA's TMA → this CTA's splitters
    auto split_bar = [&](int s) { return bars + 8u * (F_STAGES + s); };        // both CTAs' splitters → leader's MMA thread
    auto empty_bar = [&](int s) { return bars + 8u * (2 * F_STAGES + s); };    // MMA → each CTA's TMA (commit to both)
    auto tfull_bar = [&](int a) { return bars + 8u * (3 * F_STAGES + a); };
    auto tempty_bar = [&](int a) { return bars + 8u * (3 * F_STAGES + ACC_STAGES + a); };  // leader: 8 epilogue warps
    constexpr int SLOT_OFF = 8 * (3 * F_STAGES + 2 * ACC_STAGES);
    const uint32_t tmem_slot = bars + SLOT_OFF;
    volatile uint32_t *tmem_slot_ptr = reinterpret_cast<volatile uint32_t *>(gen_base + F_STAGES * F_STAGE_BYTES + SLOT_OFF);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(gen_base + F_STAGES * F_STAGE_BYTES + SLOT_OFF + 8);
    auto a_hi = [&](int s) { return smem_base + s * F_STAGE_BYTES; };
    auto b_hi = [&](int s) { return smem_base + s * F_STAGE_BYTES + F_A_BYTES; };
    auto a_lo = [&](int s) { return smem_base + s * F_STAGE_BYTES + F_RAW_BYTES; };
    auto b_lo = [&](int s) { return smem_base + s * F_STAGE_BYTES + F_RAW_BYTES + F_A_BYTES; };

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int pair = blockIdx.x >> 1;
    const int num_pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < F_STAGES; ++s) {
            mbar_init(raw_bar(s), 1);
            mbar_init(split_bar(s), 8);  // used in the leader only: 4 splitter warps × 2 CTAs
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < ACC_STAGES; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 8);  // used in the leader only
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
    }
    if (warp == 1) tmem_alloc_pair(tmem_slot, FP_TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_ptr;

    auto tile_coords = [&](int tile, int &b, int &tm, int &tn) { grouped_tile_coords(tile, p.tiles_m, p.tiles_n, p.raster, b, tm, tn); };

    if (warp == 0) {
        // ===== TMA producer: this CTA's A slice and B half, completing on this CTA's raw barrier =====
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = pair; tile < p.num_tiles && ok; tile += num_pairs) {
                int b, tm, tn;
                tile_coords(tile, b, tm, tn);
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1, abort_flag)) {
                        if (!*abort_flag) { *abort_flag = 1; atomicExch(p.status, GEMM_TIMEOUT_EMPTY); }
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(raw_bar(stage), F_RAW_BYTES);
                    tma_load_3d(a_hi(stage), &tmap_a, raw_bar(stage), kb * F_BK, tm * PBM + int(rank) * BM, b);
#pragma unroll
                    for (int j = 0; j < F_BN / F_B_BOX_N; ++j)
                        tma_load_3d(b_hi(stage) + j * F_B_BOX_BYTES, &tmap_b, raw_bar(stage),
                                    tn * FP_BN + int(rank) * F_BN + j * F_B_BOX_N, kb * F_BK, b);
                    if (++stage == F_STAGES) { stage = 0; phase ^= 1; }
                }
            }
            if (*abort_flag) {
                const long long t0 = clock64();
                while (clock64() - t0 < 2000000ll) {}
            }
        }
    } else if (warp == 1) {
        // ===== MMA issuer: one thread of the leader =====
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = make_idesc_tf32_pair();
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int tile = pair; tile < p.num_tiles && ok; tile += num_pairs) {
                if (!mbar_wait_cluster(tempty_bar(acc), acc_phase ^ 1, abort_flag)) {
                    if (!*abort_flag) { *abort_flag = 1; atomicExch(p.status, GEMM_TIMEOUT_TMEM_EMPTY); }
                    break;
                }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + acc * FP_BN;
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    if (!mbar_wait_cluster(split_bar(stage), phase, abort_flag)) {
                        if (!*abort_flag) { *abort_flag = 1; atomicExch(p.status, GEMM_TIMEOUT_SPLIT); }
                        ok = false;
                        break;
                    }
                    tc_fence_after();
#pragma unroll
                    for (int k = 0; k < F_BK / F_UMMA_K; ++k) {
                        const uint64_t ah = make_smem_desc(a_hi(stage) + k * 32, 16, 1024);
                        const uint64_t al = make_smem_desc(a_lo(stage) + k * 32, 16, 1024);
                        const uint64_t bh = make_smem_desc(b_hi(stage) + k * 1024, F_B_BOX_BYTES, 512, 1);
                        const uint64_t bl = make_smem_desc(b_lo(stage) + k * 1024, F_B_BOX_BYTES, 512, 1);
                        umma_tf32_pair(tmem_d, al, bh, idesc, (kb | k) != 0);  // small terms first
                        umma_tf32_pair(tmem_d, ah, bl, idesc, 1);
                        umma_tf32_pair(tmem_d, ah, bh, idesc, 1);
                    }
                    umma_commit_pair(empty_bar(stage), 0x3);
                    if (++stage == F_STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                umma_commit_pair(tfull_bar(acc), 0x3);
                if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1; }
            }
        }
    } else if (warp < 6) {
        // ===== epilogue: each CTA drains its own 128 rows × 256 columns =====
        const int q = warp & 3;
        int acc = 0;
        uint32_t acc_phase = 0;
        const bool vec_ok = (p.N % 4) == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0;
        for (int tile = pair; tile < p.num_tiles; tile += num_pairs) {
            int b, tm, tn;
            tile_coords(tile, b, tm, tn);
            if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag)) {
                if (lane == 0 && !*abort_flag) { *abort_flag = 1; atomicExch(p.status, GEMM_TIMEOUT_TMEM_FULL); }
                break;
            }
            tc_fence_after();
            const int row = tm * PBM + int(rank) * BM + q * 32 + lane;
            float *crow = C + (size_t(b) * p.M + row) * p.N;
#pragma unroll 1
            for (int c0 = 0; c0 < FP_BN; c0 += 32) {
                uint32_t r[32];
                tmem_ld_32x32b_x32(tmem_base + (uint32_t(q * 32) << 16) + acc * FP_BN + c0, r);
                tmem_ld_wait();
                const int col = tn * FP_BN + c0;
                if (row < p.M) {
                    if (vec_ok && col + 32 <= p.N) {
#pragma unroll
                        for (int v = 0; v < 8; ++v)
                            *reinterpret_cast<uint4 *>(crow + col + 4 * v) = make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (col + j < p.N) crow[col + j] = __uint_as_float(r[j]);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa_u32(tempty_bar(acc), 0));
            if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1; }
        }
    } else {
        // ===== splitters: warps 6..9 of BOTH CTAs; each CTA splits what its own TMA delivered =====
        const int t = threadIdx.x - 6 * 32;
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int tile = pair; tile < p.num_tiles && ok; tile += num_pairs) {
            for (int kb = 0; kb < p.k_blocks; ++kb) {
                if (!mbar_wait(raw_bar(stage), phase, abort_flag)) {
                    if (lane == 0 && !*abort_flag) { *abort_flag = 1; atomicExch(p.status, GEMM_TIMEOUT_RAW); }
                    ok = false;
                    break;
                }
                float4 *hi = reinterpret_cast<float4 *>(gen_base + stage * F_STAGE_BYTES);
                float4 *lo = reinterpret_cast<float4 *>(gen_base + stage * F_STAGE_BYTES + F_RAW_BYTES);
#pragma unroll 4
                for (int i = t; i < F_RAW_BYTES / 16; i += 128) {
                    const float4 x = hi[i];
                    float4 h, l;
                    h.x = round_tf32(x.x); l.x = x.x - h.x;
                    h.y = round_tf32(x.y); l.y = x.y - h.y;
                    h.z = round_tf32(x.z); l.z = x.z - h.z;
                    h.w = round_tf32(x.w); l.w = x.w - h.w;
                    hi[i] = h;
                    lo[i] = l;
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(mapa_u32(split_bar(stage), 0));
                if (++stage == F_STAGES) { stage = 0; phase ^= 1; }
            }
        }
    }
    // Teardown: the pair meets before either CTA leaves or frees TMEM.
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, FP_TMEM_COLS);
    }
}

// ---- SIMT FMA kernel for f32 / f64 (and shapes the TMA path cannot take) -----------------------
template <typename T, typename A, int TS, int RT>
__global__ void __launch_bounds__((TS / RT) * (TS / RT))
    gemm_simt_kernel(const T *__restrict__ Am, const T *__restrict__ Bm, T *__restrict__ Cm, int M, int N, int K) {
    constexpr int KT = 16;
    constexpr int NT = (TS / RT) * (TS / RT);
    __shared__ A sa[KT][TS + 1];
    __shared__ A sb[KT][TS + 1];
    const int b = blockIdx.z;
    Am += size_t(b) * M * K;
    Bm += size_t(b) * K * N;
    Cm += size_t(b) * M * N;
    const int tx = threadIdx.x % (TS / RT), ty = threadIdx.x / (TS / RT);
    const int m0 = blockIdx.y * TS, n0 = blockIdx.x * TS;
    A acc[RT][RT];
#pragma unroll
    for (int i = 0; i < RT; ++i)
#pragma unroll
        for (int j = 0; j < RT; ++j) acc[i][j] = A(0);
    for (int k0 = 0; k0 < K; k0 += KT) {
        for (int i = threadIdx.x; i < TS * KT; i += NT) {
            const int r = i / KT, c = i % KT;  // A tile: TS rows × KT
            sa[c][r] = (m0 + r < M && k0 + c < K) ? A(to_compute(Am[size_t(m0 + r) * K + k0 + c])) : A(0);
        }
        for (int i = threadIdx.x; i < TS * KT; i += NT) {
            const int r = i / TS, c = i % TS;  // B tile: KT rows × TS
            sb[r][c] = (k0 + r < K && n0 + c < N) ? A(to_compute(Bm[size_t(k0 + r) * N + n0 + c])) : A(0);
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < KT; ++k) {
            A av[RT], bv[RT];
#pragma unroll
            for (int i = 0; i < RT; ++i) av[i] = sa[k][ty * RT + i];
#pragma unroll
            for (int j = 0; j < RT; ++j) bv[j] = sb[k][tx * RT + j];
#pragma unroll
            for (int i = 0; i < RT; ++i)
#pragma unroll
                for (int j = 0; j < RT; ++j) acc[i][j] += av[i] * bv[j];
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < RT; ++i)
#pragma unroll
        for (int j = 0; j < RT; ++j) {
            const int m = m0 + ty * RT + i, n = n0 + tx * RT + j;
            if (m < M && n < N) Cm[size_t(m) * N + n] = from_compute<T>(static_cast<compute_t<T>>(acc[i][j]));
        }
}

template <typename T, typename A>
int launch_simt(const T *Am, const T *Bm, T *Cm, int64_t batch, int64_t M, int64_t N, int64_t K, cudaStream_t st) {
    constexpr int TS = 64, RT = 4;
    if (batch > 65535) return fail(DX_E_SHAPE, "matmul: batch %lld too large", (long long)batch);
    dim3 grid((unsigned)((N + TS - 1) / TS), (unsigned)((M + TS - 1) / TS), (unsigned)batch);
    if (grid.y > 65535) return fail(DX_E_SHAPE, "matmul: M %lld too large for the SIMT path", (long long)M);
    gemm_simt_kernel<T, A, TS, RT><<<grid, (TS / RT) * (TS / RT), 0, st>>>(Am, Bm, Cm, (int)M, (int)N, (int)K);
    return check_launch("matmul(simt)");
}

// ---- tensor maps ----------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
        else cudaGetLastError();
    });
    return fn;
}

// Rows of tiles per raster group.  With one row per group the tiles run row by row: every wave
// streams all of B against a few row-panels of A, which is the best order while B (K x N) stays
// resident in the 126 MB L2 (8192 x 4096 x 4096 bf16: 173 us against 180 us with groups of 8 and
// 190 us column by column).  When B is too large for that but A fits, the mirror image (one group
// holding every row: column by column) keeps A resident instead; when neither fits, groups of 8
// bound the working set of a wave from both sides.  DX_GEMM_RASTER overrides the choice.
int raster_group(int64_t M, int64_t N, int64_t K, int es, int64_t tiles_m) {
    static const int forced = [] {
        const char *e = std::getenv("DX_GEMM_RASTER");
        const int v = e ? std::atoi(e) : 0;
        return v >= 1 && v <= (1 << 20) ? v : 0;
    }();
    if (forced) return forced;
    const int64_t resident = int64_t(48) << 20;
    if (K * N * es <= resident) return 1;
    if (M * K * es <= resident) return (int)std::max<int64_t>(tiles_m, 1);
    return 8;
}

int make_map(CUtensorMap *map, CUtensorMapDataType dt, const void *base, uint64_t inner, uint64_t rows, uint64_t batch,
             uint32_t box_inner, uint32_t box_rows, uint32_t esize = 2,
             CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
    EncodeTiledFn enc = encode_tiled();
    if (!enc) return fail(DX_E_CUDA, "matmul: cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[3] = {inner, rows, batch};
    const cuuint64_t strides[2] = {inner * esize, inner * rows * esize};  // bytes, for dims 1 and 2
    const cuuint32_t box[3] = {box_inner, box_rows, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(map, dt, 3, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(DX_E_CUDA, "matmul: cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return DX_OK;
}

// Status word of the tensor-core kernel (0 = fine), one per device that loads the module.
__device__ int g_gemm_status = 0;
std::mutex g_setup_mu;
bool g_attr_set[64][2] = {};
int *g_status_ptr[64] = {};

// How many CTA pairs can be resident at once on `dev` (0 = the pair kernel cannot run there).
// Looked up once per device and element type; also raises the kernel's shared-memory limit.
int g_pair_slots[64][2] = {};
bool g_pair_known[64][2] = {};
template <typename T> int pair_slots(int dev) {
    const int ti = std::is_same<T, bf16>::value ? 0 : 1;
    std::lock_guard<std::mutex> lk(g_setup_mu);
    if (g_pair_known[dev][ti]) return g_pair_slots[dev][ti];
    g_pair_known[dev][ti] = true;
    g_pair_slots[dev][ti] = 0;
    if (cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM_BYTES) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2u * (unsigned)sm_count(), 1, 1);
    cfg.blockDim = dim3(G_THREADS, 1, 1);
    cfg.dynamicSmemBytes = P_SMEM_BYTES;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_tcgen05_pair_kernel<T>, &cfg) != cudaSuccess) {
        cudaGetLastError();
        n = 0;
    }
    g_pair_slots[dev][ti] = n;
    return n;
}

// Persistent single-CTA kernel at tile width BN_.
// The persistent kernels are launched with programmatic stream serialisation (common.cuh): their set-up — barriers,
// TMEM, descriptor prefetch — runs while the kernel before drains.  DX_GEMM_PDL=0 or DX_PDL=0 turns it off.
bool pdl_on() {
    static const bool on = [] { const char *e = std::getenv("DX_GEMM_PDL"); return !(e && e[0] == '0'); }();
    return on && pdl_enabled();
}

template <typename T, int BN_>
int launch_single(const CUtensorMap &ma, const CUtensorMap &mb, T *C, int64_t batch, int64_t M, int64_t N, int64_t K, bool c_staged,
                  int *status, int dev, cudaStream_t st) {
    using Cfg = TileCfg<BN_>;
    {
        static bool attr_set[64] = {};
        std::lock_guard<std::mutex> lk(g_setup_mu);
        if (!attr_set[dev]) {
            cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<T, BN_>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM);
            if (e != cudaSuccess) return fail(DX_E_CUDA, "matmul: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
            attr_set[dev] = true;
        }
    }
    GemmParams p;
    p.M = (int)M; p.N = (int)N; p.K = (int)K; p.batch = (int)batch;
    p.tiles_m = (int)((M + BM - 1) / BM);
    p.tiles_n = (int)((N + BN_ - 1) / BN_);
    const int64_t tiles = int64_t(p.tiles_m) * p.tiles_n * batch;
    if (tiles >= (1ll << 31)) return fail(DX_E_SHAPE, "matmul: too many tiles");
    p.num_tiles = (int)tiles;
    p.k_blocks = (int)((K + BK - 1) / BK);
    p.status = status;
    p.raster = raster_group(M, N, K, (int)sizeof(T), p.tiles_m);
    p.c_staged = c_staged ? 1 : 0;
    const int grid = (int)std::min<int64_t>(tiles, sm_count());
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid, 1, 1);
    cfg.blockDim = dim3(G_THREADS, 1, 1);
    cfg.dynamicSmemBytes = Cfg::SMEM;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_on() ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tcgen05_kernel<T, BN_>, ma, mb, C, p);
    if (e != cudaSuccess) return fail(DX_E_CUDA, "matmul(tcgen05): %s", cudaGetErrorString(e));
    return check_launch("matmul(tcgen05)");
}

// Cost model, in SM cycles, behind the choice of kernel and tile width; the constants are fitted to
// measurements.  What bounds the main loop is operand traffic out of L2: an SM takes in about 64 bytes
// per clock, all SMs together about 6800.  Per 64-deep K block a single CTA pulls 48 / 32 / 24 KiB for
// a 128 × 256 / 128 / 64 tile (770 / 512 / 384 cycles, more than the 512 / 256 / 128 the tensor core
// needs); the two CTAs of a pair pull 32 KiB each for a 256 × 256 tile and stay near the tensor core's
// 512.  On top comes what a tile costs besides its main loop — mostly writing C, which overlaps the
// next tile's main loop only in part: about 0.75 × (400 + bytes / 20) cycles per CTA tile, and about
// 4300 per pair tile (the pair's barriers cross SMs).  With K of a few hundred that term decides.
int64_t tiles_cost(int64_t tiles, int64_t slots, int64_t k_blocks, int64_t cycles_per_kb, int64_t bytes_per_kb, int64_t per_tile) {
    const int64_t waves = (tiles + slots - 1) / slots;
    return std::max<int64_t>(waves * (k_blocks * cycles_per_kb + per_tile), tiles * k_blocks * bytes_per_kb / 6800);
}
constexpr int64_t PAIR_TILE_OVERHEAD = 4300;
constexpr int64_t single_tile_overhead(int bn) { return (400 + int64_t(BM) * bn * 2 / 20) * 3 / 4; }
int pick_tile_n(int64_t M, int64_t N, int64_t K, int64_t batch, int64_t *cost_out = nullptr) {
    static const int forced = [] {
        const char *e = std::getenv("DX_GEMM_TILE_N");
        const int v = e ? std::atoi(e) : 0;
        return (v == 256 || v == 128 || v == 64) ? v : 0;
    }();
    const int64_t sms = sm_count(), tiles_m = (M + BM - 1) / BM, k_blocks = (K + BK - 1) / BK;
    const int widths[3] = {256, 128, 64};
    const int64_t cycles[3] = {770, 512, 384};
    int best = 256;
    int64_t best_cost = -1;
    for (int i = 0; i < 3; ++i) {
        if (forced && widths[i] != forced) continue;
        const int64_t tiles = tiles_m * ((N + widths[i] - 1) / widths[i]) * batch;
        const int64_t cost = tiles_cost(tiles, sms, k_blocks, cycles[i], A_STAGE_BYTES + int64_t(widths[i]) * BK * 2, single_tile_overhead(widths[i]));
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = widths[i]; }
    }
    if (cost_out) *cost_out = best_cost;
    return best;
}

template <typename T>
int launch_tcgen05(const T *A, const T *B, T *C, int64_t batch, int64_t M, int64_t N, int64_t K, cudaStream_t st) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return fail(DX_E_CUDA, "matmul: device index %d out of range", dev);
    int *status;
    {
        std::lock_guard<std::mutex> lk(g_setup_mu);
        if (!g_status_ptr[dev]) {
            void *sym = nullptr;
            cudaError_t e = cudaGetSymbolAddress(&sym, g_gemm_status);
            if (e != cudaSuccess) return fail(DX_E_CUDA, "matmul: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
            g_status_ptr[dev] = static_cast<int *>(sym);
        }
        status = g_status_ptr[dev];
    }
    const CUtensorMapDataType dt = std::is_same<T, bf16>::value ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUtensorMap ma, mb;
    if (int e = make_map(&ma, dt, A, (uint64_t)K, (uint64_t)M, (uint64_t)batch, BK, BM)) return e;
    if (int e = make_map(&mb, dt, B, (uint64_t)N, (uint64_t)K, (uint64_t)batch, B_BOX_N, BK)) return e;
    // 16-byte stores into C need its base aligned (its pitch is: N % 8 == 0 on this path); DX_GEMM_STAGED_STORE=0 turns them off
    static const bool staged_on = [] { const char *e = std::getenv("DX_GEMM_STAGED_STORE"); return !(e && e[0] == '0'); }();
    const bool c_staged = staged_on && aligned_to(C, 16);

    // ---- CTA-pair form: worth it once there is at least one 256 × 256 tile per pair of SMs ----
    const int64_t ptiles_m = (M + PBM - 1) / PBM, ptiles_n = (N + BN - 1) / BN;
    const int64_t ptiles = ptiles_m * ptiles_n * batch;
    const int pairs = pair_slots<T>(dev);
    int mode = -1;  // auto
    if (const char *env = std::getenv("DX_GEMM_CTA_PAIR")) mode = (env[0] == '1') ? 1 : (env[0] == '0' ? 0 : -1);
    int64_t single_cost = 0;
    const int tile_n = pick_tile_n(M, N, K, batch, &single_cost);
    const int64_t k_blocks_all = (K + BK - 1) / BK;
    const bool pair_cheaper = pairs > 0 && tiles_cost(ptiles, pairs, k_blocks_all, 550, 2 * P_STAGE_BYTES, PAIR_TILE_OVERHEAD) <= single_cost;
    const bool use_pair = pairs > 0 && ptiles < (1ll << 31) && (mode == 1 || (mode == -1 && pair_cheaper));
    if (use_pair) {
        PairParams pp;
        pp.M = (int)M; pp.N = (int)N; pp.K = (int)K; pp.batch = (int)batch;
        pp.tiles_m = (int)ptiles_m;
        pp.tiles_n = (int)ptiles_n;
        pp.num_tiles = (int)ptiles;
        pp.k_blocks = (int)((K + BK - 1) / BK);
        pp.status = status;
        pp.raster = raster_group(M, N, K, (int)sizeof(*A), ptiles_m);
        pp.c_staged = c_staged ? 1 : 0;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2u * (unsigned)std::min<int64_t>(ptiles, pairs), 1, 1);
        cfg.blockDim = dim3(G_THREADS, 1, 1);
        cfg.dynamicSmemBytes = P_SMEM_BYTES;
        cfg.stream = st;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = pdl_on() ? 2 : 1;
        cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tcgen05_pair_kernel<T>, ma, mb, C, pp);
        if (e != cudaSuccess) return fail(DX_E_CUDA, "matmul(tcgen05 pair): %s", cudaGetErrorString(e));
        return check_launch("matmul(tcgen05 pair)");
    }
    switch (tile_n) {
        case 64: return launch_single<T, 64>(ma, mb, C, batch, M, N, K, c_staged, status, dev, st);
        case 128: return launch_single<T, 128>(ma, mb, C, batch, M, N, K, c_staged, status, dev, st);
        default: return launch_single<T, 256>(ma, mb, C, batch, M, N, K, c_staged, status, dev, st);
    }
}

// Few rows: the split-K cluster kernel.  DX_E_UNSUPPORTED = not a shape for it.
template <typename T> int launch_splitk(const T *A, const T *B, T *C, int64_t batch, int64_t M, int64_t N, int64_t K, cudaStream_t st) {
    if (M > BM || batch > 65535) return DX_E_UNSUPPORTED;
    const int64_t tiles_n = (N + S_BN - 1) / S_BN;
    const int64_t k_blocks = (K + BK - 1) / BK;
    // worth it only where the persistent kernels would leave most SMs idle
    const int64_t big_tiles = ((N + BN - 1) / BN) * batch;
    if (big_tiles * 2 > sm_count() || k_blocks < 8 || tiles_n * 8 >= (1ll << 31)) return DX_E_UNSUPPORTED;
    int cs = 1;
    while (cs < 8 && tiles_n * batch * cs * 2 <= 2 * sm_count() && k_blocks / (cs * 2) >= 4) cs *= 2;  // two CTAs per SM: stay within one wave
    bool forced = false;
    if (const char *e = std::getenv("DX_GEMM_SPLITK_CS")) {  // tuning override: 2, 4 or 8 K slices
        const int v = std::atoi(e);
        if ((v == 2 || v == 4 || v == 8) && k_blocks / v >= 1) { cs = v; forced = true; }
    }
    if (cs < 4 && !forced) return DX_E_UNSUPPORTED;  // measured: with fewer than four K slices per tile the persistent kernels are as fast
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return fail(DX_E_CUDA, "matmul: device index %d out of range", dev);
    int *status;
    {
        std::lock_guard<std::mutex> lk(g_setup_mu);
        if (!g_status_ptr[dev]) {
            void *sym = nullptr;
            cudaError_t e = cudaGetSymbolAddress(&sym, g_gemm_status);
            if (e != cudaSuccess) return fail(DX_E_CUDA, "matmul: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
            g_status_ptr[dev] = static_cast<int *>(sym);
        }
        status = g_status_ptr[dev];
        static bool attr_set[64][2] = {};
        const int ti = std::is_same<T, bf16>::value ? 0 : 1;
        if (!attr_set[dev][ti]) {
            cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_splitk_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, S_SMEM_BYTES);
            if (e != cudaSuccess) return fail(DX_E_CUDA, "matmul: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
            // two CTAs of 97 KiB per SM need the large shared-memory split of the L1
            cudaFuncSetAttribute(gemm_tcgen05_splitk_kernel<T>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
            cudaGetLastError();
            attr_set[dev][ti] = true;
        }
    }
    const CUtensorMapDataType dt = std::is_same<T, bf16>::value ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUtensorMap ma, mb;
    if (int e = make_map(&ma, dt, A, (uint64_t)K, (uint64_t)M, (uint64_t)batch, BK, BM)) return e;
    if (int e = make_map(&mb, dt, B, (uint64_t)N, (uint64_t)K, (uint64_t)batch, B_BOX_N, BK)) return e;
    SplitKParams p;
    p.M = (int)M; p.N = (int)N; p.K = (int)K; p.batch = (int)batch;
    p.tiles_n = (int)tiles_n;
    p.k_blocks = (int)k_blocks;
    p.kb_per_rank = (int)((k_blocks + cs - 1) / cs);
    p.status = status;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(tiles_n * cs), (unsigned)batch, 1);
    cfg.blockDim = dim3(NUM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = S_SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cs;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tcgen05_splitk_kernel<T>, ma, mb, C, p);
    if (e != cudaSuccess) return fail(DX_E_CUDA, "matmul(tcgen05 split-K): %s", cudaGetErrorString(e));
    return check_launch("matmul(tcgen05 split-K)");
}

// A few rows of 256 x 256 tiles: K split over the pairs of a cluster.  DX_E_UNSUPPORTED = not a shape for it.
// How many clusters of 2·ks CTAs of the pair split-K kernel the device runs at once (0 = none): the CTAs
// of a cluster must sit in one GPC, which caps it well below SMs / cluster size.  Looked up once.
template <typename T> int pair_splitk_clusters(int dev, int ks) {
    static int known[64][2][2] = {};  // 0 unknown, else clusters + 1
    const int ti = std::is_same<T, bf16>::value ? 0 : 1, ci = ks == 2 ? 0 : 1;
    std::lock_guard<std::mutex> lk(g_setup_mu);
    if (known[dev][ti][ci] == 0) {
        int n = 0;
        if (cudaFuncSetAttribute(gemm_tcgen05_pair_splitk_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, PS_SMEM_BYTES) == cudaSuccess) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3((unsigned)(2 * ks * sm_count()), 1, 1);
            cfg.blockDim = dim3(NUM_THREADS, 1, 1);
            cfg.dynamicSmemBytes = PS_SMEM_BYTES;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = (unsigned)(2 * ks);
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            if (cudaOccupancyMaxActiveClusters(&n, gemm_tcgen05_pair_splitk_kernel<T>, &cfg) != cudaSuccess) n = 0;
        }
        if (n <= 0) { n = 0; cudaGetLastError(); }
        known[dev][ti][ci] = n + 1;
    }
    return known[dev][ti][ci] - 1;
}

// A few rows of 256 x 256 tiles: K split over the pairs of a cluster.  DX_E_UNSUPPORTED = not a shape for it.
template <typename T>
int launch_pair_splitk(const T *A, const T *B, T *C, int64_t batch, int64_t M, int64_t N, int64_t K, cudaStream_t st) {
    const int64_t tiles_m = (M + PBM - 1) / PBM, tiles_n = (N + BN - 1) / BN;
    const int64_t tiles = tiles_m * tiles_n * batch;
    const int64_t k_blocks = (K + BK - 1) / BK;
    if (M <= BM || tiles * 2 > sm_count() / 2) return DX_E_UNSUPPORTED;  // one row of tiles, or enough tiles for the persistent kernels
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return fail(DX_E_CUDA, "matmul: device index %d out of range", dev);
    // the widest split whose clusters all run at once and whose slices keep at least 48 K blocks: the two
    // cluster barriers, the push and the late start cost about as much as 30 K blocks of main loop
    // (DX_GEMM_PAIR_SPLITK=2|4 forces that many slices wherever the clusters fit and every slice gets a K block)
    int forced = 0;
    if (const char *e = std::getenv("DX_GEMM_PAIR_SPLITK")) forced = (e[0] == '2' || e[0] == '4') ? e[0] - '0' : 0;
    int ks = 0;
    if (forced) {
        if (k_blocks >= forced && tiles <= pair_splitk_clusters<T>(dev, forced)) ks = forced;
    } else {
        for (int cand = 4; cand >= 2 && !ks; cand >>= 1)
            if (k_blocks / cand >= 48 && tiles <= pair_splitk_clusters<T>(dev, cand)) ks = cand;
    }
    if (!ks) return DX_E_UNSUPPORTED;
    int *status;
    {
        std::lock_guard<std::mutex> lk(g_setup_mu);
        if (!g_status_ptr[dev]) {
            void *sym = nullptr;
            cudaError_t e = cudaGetSymbolAddress(&sym, g_gemm_status);
            if (e != cudaSuccess) return fail(DX_E_CUDA, "matmul: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
            g_status_ptr[dev] = static_cast<int *>(sym);
        }
        status = g_status_ptr[dev];
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(tiles * ks * 2), 1, 1);
    cfg.blockDim = dim3(NUM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = PS_SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)(ks * 2);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const CUtensorMapDataType dt = std::is_same<T, bf16>::value ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUtensorMap ma, mb;
    if (int e = make_map(&ma, dt, A, (uint64_t)K, (uint64_t)M, (uint64_t)batch, BK, BM)) return e;
    if (int e = make_map(&mb, dt, B, (uint64_t)N, (uint64_t)K, (uint64_t)batch, B_BOX_N, BK)) return e;
    PairSplitParams p;
    p.M = (int)M; p.N = (int)N; p.K = (int)K; p.batch = (int)batch;
    p.tiles_m = (int)tiles_m;
    p.tiles_n = (int)tiles_n;
    p.k_blocks = (int)k_blocks;
    p.kb_per_slice = (int)((k_blocks + ks - 1) / ks);
    p.status = status;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tcgen05_pair_splitk_kernel<T>, ma, mb, C, p);
    if (e != cudaSuccess) return fail(DX_E_CUDA, "matmul(tcgen05 pair split-K): %s", cudaGetErrorString(e));
    return check_launch("matmul(tcgen05 pair split-K)");
}

// A few rows of 256 x 256 tiles, K split over independent pairs through the caller's workspace.
// plan: how many K slices (0 = not a shape for it) and the workspace that needs.
unsigned long long *g_wsk_counter_ptr[64] = {};
// Launches of this kernel on different streams may overlap, and each needs counters of its own: a stream gets a bank
// the first time it launches the kernel and keeps it.  -1: all banks belong to other streams (the other kernels run).
std::vector<cudaStream_t> g_wsk_bank_streams[64];
int wsk_bank(int dev, cudaStream_t st) {  // caller holds g_setup_mu
    auto &v = g_wsk_bank_streams[dev];
    for (size_t i = 0; i < v.size(); ++i)
        if (v[i] == st) return int(i);
    if (v.size() >= size_t(WSK_BANKS)) return -1;
    v.push_back(st);
    return int(v.size()) - 1;
}
template <typename T> int pair_wsk_slots(int dev) {
    static int known[64][2] = {};  // 0 unknown, else clusters + 1
    const int ti = std::is_same<T, bf16>::value ? 0 : 1;
    std::lock_guard<std::mutex> lk(g_setup_mu);
    if (known[dev][ti] == 0) {
        int n = 0;
        if (cudaFuncSetAttribute(gemm_tcgen05_pair_wsk_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, PS_SMEM_BYTES) == cudaSuccess) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3((unsigned)(2 * sm_count()), 1, 1);
            cfg.blockDim = dim3(W_THREADS, 1, 1);
            cfg.dynamicSmemBytes = PS_SMEM_BYTES;
            cudaLaunchAttribute attr[2];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 2;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            attr[1].id = cudaLaunchAttributeCooperative;
            attr[1].val.cooperative = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 2;
            if (cudaOccupancyMaxActiveClusters(&n, gemm_tcgen05_pair_wsk_kernel<T>, &cfg) != cudaSuccess) n = 0;
        }
        if (n <= 0) { n = 0; cudaGetLastError(); }
        known[dev][ti] = n + 1;
    }
    return known[dev][ti] - 1;
}

// K slices for a shape (0: the other kernels do it), given how many pairs run at once.
int wsk_slices(int64_t batch, int64_t M, int64_t N, int64_t K, int slots) {
    static const int forced = [] {  // DX_GEMM_WSK=0 turns the path off, 2..8 forces that many slices where they fit
        const char *e = std::getenv("DX_GEMM_WSK");
        return e ? std::atoi(e) : -1;
    }();
    if (forced == 0 || slots <= 0 || M <= BM) return 0;
    const int64_t tiles = ((M + PBM - 1) / PBM) * ((N + BN - 1) / BN) * batch;
    const int64_t k_blocks = (K + BK - 1) / BK;
    if (tiles * 2 > slots || tiles * 2 > 512) return 0;  // enough tiles for the persistent kernels (or more than there are counters)
    int64_t ks = std::min<int64_t>(std::min<int64_t>(8, slots / tiles), k_blocks / 4);
    if (forced >= 2) ks = std::min<int64_t>(std::min<int64_t>(forced, 8), std::min<int64_t>(slots / tiles, k_blocks));
    while (ks >= 2 && (ks - 1) * ((k_blocks + ks - 1) / ks) >= k_blocks) --ks;  // no slice without a K block
    if (ks < 2) return 0;
    // What splitting saves in main-loop time has to outweigh what the exchange costs: storing the blocks other pairs
    // finish (an SM pushes about 32 bytes per clock into L2), the release, the count-in and the wait for the slowest
    // pair (three trips to L2, about 1.5 µs), reading the others' blocks and the larger launch — together some 5 µs,
    // i.e. about 18 K blocks of main loop.  Measured, bf16, µs without -> with the split: 512 x 4096 x 4096 24.1 ->
    // 18.5, 256 x 4096 x 4096 22.3 -> 14.4, 768 x 2048 x 8192 32.5 -> 23.5, 256 x 1024 x 16384 33.3 -> 19.8,
    // 300 x 520 x 8008 36.2 -> 16.5, 512 x 2048 x 2048 13.0 -> 11.9, but 1024^3 (12 blocks saved) 8.1 -> 10.5.
    if (forced < 2 && k_blocks * (ks - 1) / ks < 20) return 0;
    return int(ks);
}

template <typename T>
int launch_pair_wsk(const T *A, const T *B, T *C, int64_t batch, int64_t M, int64_t N, int64_t K, void *ws, size_t ws_bytes, cudaStream_t st) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return fail(DX_E_CUDA, "matmul: device index %d out of range", dev);
    const int ks = wsk_slices(batch, M, N, K, pair_wsk_slots<T>(dev));
    if (!ks) return DX_E_UNSUPPORTED;
    const int64_t tiles_m = (M + PBM - 1) / PBM, tiles_n = (N + BN - 1) / BN;
    const int64_t tiles = tiles_m * tiles_n * batch;
    const size_t need = size_t(tiles) * ks * 2 * WS_HALF_FLOATS * sizeof(float);
    if (!ws || ws_bytes < need || !aligned_to(ws, 16)) return DX_E_UNSUPPORTED;  // the caller gave no (or too little) workspace: the other kernels
    int *status;
    unsigned long long *counters;
    {
        std::lock_guard<std::mutex> lk(g_setup_mu);
        if (!g_status_ptr[dev]) {
            void *sym = nullptr;
            cudaError_t e = cudaGetSymbolAddress(&sym, g_gemm_status);
            if (e != cudaSuccess) return fail(DX_E_CUDA, "matmul: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
            g_status_ptr[dev] = static_cast<int *>(sym);
        }
        status = g_status_ptr[dev];
        if (!g_wsk_counter_ptr[dev]) {
            void *sym = nullptr;
            cudaError_t e = cudaGetSymbolAddress(&sym, g_wsk_counters);
            if (e != cudaSuccess) return fail(DX_E_CUDA, "matmul: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
            g_wsk_counter_ptr[dev] = static_cast<unsigned long long *>(sym);
        }
        const int bank = wsk_bank(dev, st);
        if (bank < 0) return DX_E_UNSUPPORTED;
        counters = g_wsk_counter_ptr[dev] + size_t(bank) * 512;
    }
    const CUtensorMapDataType dt = std::is_same<T, bf16>::value ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUtensorMap ma, mb;
    if (int e = make_map(&ma, dt, A, (uint64_t)K, (uint64_t)M, (uint64_t)batch, BK, BM)) return e;
    if (int e = make_map(&mb, dt, B, (uint64_t)N, (uint64_t)K, (uint64_t)batch, B_BOX_N, BK)) return e;
    static const bool staged_on = [] { const char *e = std::getenv("DX_GEMM_STAGED_STORE"); return !(e && e[0] == '0'); }();
    const int64_t k_blocks = (K + BK - 1) / BK;
    PairWsParams p;
    p.M = (int)M; p.N = (int)N; p.K = (int)K; p.batch = (int)batch;
    p.tiles_m = (int)tiles_m;
    p.tiles_n = (int)tiles_n;
    p.k_blocks = (int)k_blocks;
    p.ks = ks;
    p.kb_per_slice = (int)((k_blocks + ks - 1) / ks);
    p.c_staged = (staged_on && aligned_to(C, 16)) ? 1 : 0;
    p.status = status;
    p.partial = static_cast<float *>(ws);
    p.counters = counters;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(tiles * ks * 2), 1, 1);
    cfg.blockDim = dim3(W_THREADS, 1, 1);
    cfg.dynamicSmemBytes = PS_SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeCooperative;  // the pairs of a tile wait for one another: all of them must be resident
    attr[1].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tcgen05_pair_wsk_kernel<T>, ma, mb, C, p);
    if (e == cudaErrorCooperativeLaunchTooLarge || e == cudaErrorLaunchOutOfResources) {
        cudaGetLastError();          // fewer SMs are free for a cooperative grid than the occupancy query saw (a profiler,
        return DX_E_UNSUPPORTED;     // another context): the kernels without a K split take the call
    }
    if (e != cudaSuccess) return fail(DX_E_CUDA, "matmul(tcgen05 pair, K split through the workspace): %s", cudaGetErrorString(e));
    return check_launch("matmul(tcgen05 pair, K split through the workspace)");
}

// float32 through the tensor cores (three TF32 products per product).
bool g_tf32_attr[64] = {};
int g_tf32_pair_slots[64] = {};
bool g_tf32_pair_known[64] = {};
// Resident CTA pairs of the float32 pair kernel on `dev` (0 = it cannot run there).
int tf32_pair_slots(int dev) {
    std::lock_guard<std::mutex> lk(g_setup_mu);
    if (g_tf32_pair_known[dev]) return g_tf32_pair_slots[dev];
    g_tf32_pair_known[dev] = true;
    g_tf32_pair_slots[dev] = 0;
    if (cudaFuncSetAttribute(gemm_tf32x3_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, F_SMEM_BYTES) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2u * (unsigned)sm_count(), 1, 1);
    cfg.blockDim = dim3(F_THREADS, 1, 1);
    cfg.dynamicSmemBytes = F_SMEM_BYTES;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_tf32x3_pair_kernel, &cfg) != cudaSuccess) {
        cudaGetLastError();
        n = 0;
    }
    g_tf32_pair_slots[dev] = n;
    return n;
}
int launch_tf32x3(const float *A, const float *B, float *C, int64_t batch, int64_t M, int64_t N, int64_t K, cudaStream_t st) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return fail(DX_E_CUDA, "matmul: device index %d out of range", dev);
    int *status;
    {
        std::lock_guard<std::mutex> lk(g_setup_mu);
        if (!g_status_ptr[dev]) {
            void *sym = nullptr;
            cudaError_t e = cudaGetSymbolAddress(&sym, g_gemm_status);
            if (e != cudaSuccess) return fail(DX_E_CUDA, "matmul: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
            g_status_ptr[dev] = static_cast<int *>(sym);
        }
        status = g_status_ptr[dev];
        if (!g_tf32_attr[dev]) {
            cudaError_t e = cudaFuncSetAttribute(gemm_tf32x3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, F_SMEM_BYTES);
            if (e != cudaSuccess) return fail(DX_E_CUDA, "matmul: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
            g_tf32_attr[dev] = true;
        }
    }
    CUtensorMap ma, mb;
    if (int e = make_map(&ma, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, A, (uint64_t)K, (uint64_t)M, (uint64_t)batch, F_BK, BM, 4)) return e;
    if (int e = make_map(&mb, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, B, (uint64_t)N, (uint64_t)K, (uint64_t)batch, F_B_BOX_N, F_BK, 4,
                         CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)) return e;
    // ---- CTA-pair form: once there is at least one 256 × 256 tile per resident pair ----
    const int64_t ptiles_m = (M + PBM - 1) / PBM, ptiles_n = (N + FP_BN - 1) / FP_BN;
    const int64_t ptiles = ptiles_m * ptiles_n * batch;
    const int pairs = tf32_pair_slots(dev);
    int mode = -1;
    if (const char *env = std::getenv("DX_GEMM_CTA_PAIR")) mode = (env[0] == '1') ? 1 : (env[0] == '0' ? 0 : -1);
    if (pairs > 0 && ptiles < (1ll << 31) && (mode == 1 || (mode == -1 && ptiles >= pairs))) {
        PairParams pp;
        pp.M = (int)M; pp.N = (int)N; pp.K = (int)K; pp.batch = (int)batch;
        pp.tiles_m = (int)ptiles_m;
        pp.tiles_n = (int)ptiles_n;
        pp.num_tiles = (int)ptiles;
        pp.k_blocks = (int)((K + F_BK - 1) / F_BK);
        pp.status = status;
        pp.raster = raster_group(M, N, K, (int)sizeof(*A), ptiles_m);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2u * (unsigned)std::min<int64_t>(ptiles, pairs), 1, 1);
        cfg.blockDim = dim3(F_THREADS, 1, 1);
        cfg.dynamicSmemBytes = F_SMEM_BYTES;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tf32x3_pair_kernel, ma, mb, C, pp);
        if (e != cudaSuccess) return fail(DX_E_CUDA, "matmul(tf32x3 pair): %s", cudaGetErrorString(e));
        return check_launch("matmul(tf32x3 pair)");
    }

    GemmParams p;
    p.M = (int)M; p.N = (int)N; p.K = (int)K; p.batch = (int)batch;
    p.tiles_m = (int)((M + BM - 1) / BM);
    p.tiles_n = (int)((N + F_BN - 1) / F_BN);
    const int64_t tiles = int64_t(p.tiles_m) * p.tiles_n * batch;
    if (tiles >= (1ll << 31)) return fail(DX_E_SHAPE, "matmul: too many tiles");
    p.num_tiles = (int)tiles;
    p.k_blocks = (int)((K + F_BK - 1) / F_BK);
    p.status = status;
    p.raster = raster_group(M, N, K, (int)sizeof(*A), p.tiles_m);
    const int grid = (int)std::min<int64_t>(tiles, sm_count());
    gemm_tf32x3_kernel<<<grid, F_THREADS, F_SMEM_BYTES, st>>>(ma, mb, C, p);
    return check_launch("matmul(tf32x3)");
}

}  // namespace
}  // namespace dx

namespace dx {
int matmul_skinny(int dtype, const void *A, const void *B, void *C, int64_t batch, int64_t M, int64_t N, int64_t K, cudaStream_t st);
}
using namespace dx;

// Reads and clears the status word the tensor-core kernel writes when a bounded wait expires.
// Synchronises the stream; meant for tests and for the executor's error path.
extern "C" int dx_matmul_status(void *stream) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !g_status_ptr[dev]) return 0;
    int h = 0;
    cudaStream_t st = as_stream(stream);
    if (cudaMemcpyAsync(&h, g_status_ptr[dev], sizeof(int), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
        cudaStreamSynchronize(st) != cudaSuccess)
        return fail(DX_E_CUDA, "matmul: cannot read the status word: %s", cudaGetErrorString(cudaGetLastError()));
    if (h != 0) {
        cudaMemsetAsync(g_status_ptr[dev], 0, sizeof(int), st);
        if (g_wsk_counter_ptr[dev]) cudaMemsetAsync(g_wsk_counter_ptr[dev], 0, sizeof(unsigned long long) * WSK_BANKS * 512, st);  // a K-split launch that gave up may have left its counts behind
        return fail(DX_E_CUDA, "matmul: tensor-core pipeline wait %d expired", h);
    }
    return DX_OK;
}

extern "C" size_t dx_matmul_workspace_bytes(int dtype, int64_t batch, int64_t M, int64_t N, int64_t K) {
    if ((dtype != DX_BF16 && dtype != DX_F16) || batch <= 0 || M <= 0 || N <= 0 || K <= 0 || (K % 8) || (N % 8)) return 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); return 0; }
    const int slots = dtype == DX_BF16 ? pair_wsk_slots<bf16>(dev) : pair_wsk_slots<f16>(dev);
    const int ks = wsk_slices(batch, M, N, K, slots);
    if (!ks) return 0;
    const int64_t tiles = ((M + PBM - 1) / PBM) * ((N + BN - 1) / BN) * batch;
    return size_t(tiles) * ks * 2 * WS_HALF_FLOATS * sizeof(float);
}

extern "C" int dx_matmul(int dtype, const void *A, const void *B, void *C, int64_t batch, int64_t M, int64_t N, int64_t K,
                         void *stream) {
    return dx_matmul_ws(dtype, A, B, C, batch, M, N, K, nullptr, 0, stream);
}

extern "C" int dx_matmul_ws(int dtype, const void *A, const void *B, void *C, int64_t batch, int64_t M, int64_t N, int64_t K,
                            void *workspace, size_t workspace_bytes, void *stream) {
    cudaStream_t st = as_stream(stream);
    if (batch < 0 || M < 0 || N < 0 || K < 0) return fail(DX_E_SHAPE, "matmul: negative extent");
    if (batch == 0 || M == 0 || N == 0) return DX_OK;
    if (!A || !B || !C) {
        if (K == 0 && C) { /* fallthrough to zero fill */ } else return fail(DX_E_ARG, "matmul: null pointer");
    }
    if (M >= (1ll << 31) || N >= (1ll << 31) || K >= (1ll << 31)) return fail(DX_E_SHAPE, "matmul: extent too large");
    if (K == 0) return dx_fill(dtype, C, 0.0, 0, batch * M * N, stream);
    if (M <= 16) {
        // a handful of rows: reading B once is all the work — the streaming kernel (DX_GEMM_SKINNY=0 turns it off)
        static const bool skinny_on = [] { const char *e = std::getenv("DX_GEMM_SKINNY"); return !(e && e[0] == '0'); }();
        if (skinny_on) {
            const int rc = matmul_skinny(dtype, A, B, C, batch, M, N, K, st);
            if (rc != DX_E_UNSUPPORTED) return rc;
        }
    }
    switch (dtype) {
        case DX_BF16:
        case DX_F16: {
            // TMA needs 16-byte aligned bases and row pitches; anything else takes the SIMT path.
            const bool tma_ok = (K % 8 == 0) && (N % 8 == 0) && aligned_to(A, 16) && aligned_to(B, 16);
            if (tma_ok && M <= BM) {
                static const bool splitk_on = [] { const char *e = std::getenv("DX_GEMM_SPLITK"); return !(e && e[0] == '0'); }();
                if (splitk_on) {
                    const int rc = dtype == DX_BF16 ? launch_splitk<bf16>((const bf16 *)A, (const bf16 *)B, (bf16 *)C, batch, M, N, K, st)
                                                    : launch_splitk<f16>((const f16 *)A, (const f16 *)B, (f16 *)C, batch, M, N, K, st);
                    if (rc != DX_E_UNSUPPORTED) return rc;
                }
            }
            if (tma_ok && M > BM && workspace) {
                const int rc = dtype == DX_BF16 ? launch_pair_wsk<bf16>((const bf16 *)A, (const bf16 *)B, (bf16 *)C, batch, M, N, K, workspace, workspace_bytes, st)
                                                : launch_pair_wsk<f16>((const f16 *)A, (const f16 *)B, (f16 *)C, batch, M, N, K, workspace, workspace_bytes, st);
                if (rc != DX_E_UNSUPPORTED) return rc;
            }
            if (tma_ok && M > BM) {
                const char *psplit_env = std::getenv("DX_GEMM_PAIR_SPLITK");
                if (!(psplit_env && psplit_env[0] == '0')) {
                    const int rc = dtype == DX_BF16 ? launch_pair_splitk<bf16>((const bf16 *)A, (const bf16 *)B, (bf16 *)C, batch, M, N, K, st)
                                                    : launch_pair_splitk<f16>((const f16 *)A, (const f16 *)B, (f16 *)C, batch, M, N, K, st);
                    if (rc != DX_E_UNSUPPORTED) return rc;
                }
            }
            if (tma_ok) {
                return dtype == DX_BF16 ? launch_tcgen05<bf16>((const bf16 *)A, (const bf16 *)B, (bf16 *)C, batch, M, N, K, st)
                                        : launch_tcgen05<f16>((const f16 *)A, (const f16 *)B, (f16 *)C, batch, M, N, K, st);
            }
            return dtype == DX_BF16 ? launch_simt<bf16, float>((const bf16 *)A, (const bf16 *)B, (bf16 *)C, batch, M, N, K, st)
                                    : launch_simt<f16, float>((const f16 *)A, (const f16 *)B, (f16 *)C, batch, M, N, K, st);
        }
        case DX_F32: {
            // tensor-core path needs 16-byte aligned bases and row pitches; DX_GEMM_F32_SIMT=1 forces the FMA kernel
            const char *env = std::getenv("DX_GEMM_F32_SIMT");
            const bool tma_ok = (K % 4 == 0) && (N % 4 == 0) && aligned_to(A, 16) && aligned_to(B, 16) && !(env && env[0] == '1');
            if (tma_ok) return launch_tf32x3((const float *)A, (const float *)B, (float *)C, batch, M, N, K, st);
            return launch_simt<float, float>((const float *)A, (const float *)B, (float *)C, batch, M, N, K, st);
        }
        case DX_F64: return launch_simt<double, double>((const double *)A, (const double *)B, (double *)C, batch, M, N, K, st);
        default: return fail(DX_E_DTYPE, "matmul: unsupported dtype code %d (float dtypes only)", dtype);
    }
}
