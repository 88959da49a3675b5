// matmul with few rows of A (M <= 16): C[M,N] = A[M,K] · B[K,N], the shape of one decoding step.
//
// With so few rows the work is reading B once: K·N elements against 2·M·K·N flops, far below the
// point where tensor cores matter, so this is a streaming kernel, bound by HBM like the elementwise
// ops, not a tile GEMM (whose 128-row tiles would waste the tensor cores and — worse — put only
// N/256 CTAs on 148 SMs).  The reference calls cublasSgemm for every shape
// (executor/op-cuda/src/deepx/tensorfunc/matmul_cublas.hpp:16-78).
//
//   * a CTA owns a strip of W = 32·NC columns of B and one K-slice; a cluster of CS CTAs covers K
//     for the strip, so there are strips × CS CTAs (enough to pull full bandwidth even for N = 4096);
//   * thread (lane, kl): NC consecutive columns (one 8- or 16-byte load per row of B), rows
//     k ≡ kl (mod 8) of the slice, U rows in flight; A's slice sits in shared memory and is read
//     as a broadcast; M × NC fp32 accumulators per thread;
//   * the 8 row-lanes of a CTA are combined through shared memory, the CS CTAs of the cluster through
//     distributed shared memory, both in a fixed order (no atomics, no workspace, same bits every run).
#include <cstdlib>
#include <mutex>

#include "common.cuh"

namespace dx {
namespace {

constexpr int SK_THREADS = 256;
constexpr int SK_KL = 8;   // row lanes per CTA
constexpr int SK_U = 8;    // rows of B in flight per thread

__device__ __forceinline__ uint32_t sk_cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t sk_cluster_size() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void sk_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float sk_ld_remote(const float *local, uint32_t rank) {
    const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(local));
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(rank));
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(r) : "memory");
    return v;
}

struct SkinnyParams {
    int M, N, K;
    int kchunk;  // rows of B per cluster rank (multiple of SK_KL)
};

template <typename T, int MT, int NC>
__global__ void __launch_bounds__(SK_THREADS) gemm_skinny_kernel(const T *__restrict__ A, const T *__restrict__ B, T *__restrict__ C, SkinnyParams p) {
    constexpr int W = 32 * NC;
    extern __shared__ __align__(16) unsigned char sk_smem[];
    float *red = reinterpret_cast<float *>(sk_smem);               // [SK_KL / 2][MT][W]
    T *sA = reinterpret_cast<T *>(sk_smem + size_t(SK_KL / 2) * MT * W * sizeof(float));  // [MT][kchunk]
    const int lane = threadIdx.x & 31, kl = threadIdx.x >> 5;
    const uint32_t rank = sk_cluster_rank(), cs = sk_cluster_size();
    const int strip = blockIdx.x / cs;
    const int64_t batch = blockIdx.y;
    A += batch * int64_t(p.M) * p.K;
    B += batch * int64_t(p.K) * p.N;
    C += batch * int64_t(p.M) * p.N;
    const int k0 = int(rank) * p.kchunk;
    const int k1 = min(p.K, k0 + p.kchunk);
    const int n0 = strip * W + lane * NC;
    const bool live = n0 < p.N;  // N is a multiple of NC: a thread's columns are all in or all out

    // A's slice → shared memory (zero beyond M or K)
    for (int i = threadIdx.x; i < MT * p.kchunk; i += SK_THREADS) {
        const int m = i / p.kchunk, k = k0 + (i - m * p.kchunk);
        sA[i] = (m < p.M && k < k1) ? A[int64_t(m) * p.K + k] : from_compute<T>(compute_t<T>(0));
    }
    __syncthreads();

    float acc[MT][NC];
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int j = 0; j < NC; ++j) acc[m][j] = 0.f;
    if (live) {
        for (int k = k0 + kl; k < k1; k += SK_KL * SK_U) {
            Pack<T, NC> b[SK_U];
#pragma unroll
            for (int u = 0; u < SK_U; ++u) {
                const int kk = k + u * SK_KL;
                if (kk < k1) b[u] = ld_stream<T, NC>(B + int64_t(kk) * p.N + n0);
            }
#pragma unroll
            for (int u = 0; u < SK_U; ++u) {
                const int kk = k + u * SK_KL;
                if (kk < k1) {
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        const float a = float(to_compute(sA[m * p.kchunk + (kk - k0)]));
#pragma unroll
                        for (int j = 0; j < NC; ++j) acc[m][j] = fmaf(a, float(to_compute(b[u].v[j])), acc[m][j]);
                    }
                }
            }
        }
    }
    // the 8 row lanes of the CTA, pairwise: lanes 4-7 into 0-3, 2-3 into 0-1, 1 into 0
#pragma unroll
    for (int half = SK_KL / 2; half >= 1; half >>= 1) {
        if (kl >= half && kl < 2 * half) {
#pragma unroll
            for (int m = 0; m < MT; ++m)
#pragma unroll
                for (int j = 0; j < NC; ++j) red[((kl - half) * MT + m) * W + lane * NC + j] = acc[m][j];
        }
        __syncthreads();
        if (kl < half) {
#pragma unroll
            for (int m = 0; m < MT; ++m)
#pragma unroll
                for (int j = 0; j < NC; ++j) acc[m][j] += red[(kl * MT + m) * W + lane * NC + j];
        }
        __syncthreads();
    }
    // this CTA's partial → red[0..MT), then the cluster's ranks in order
    if (kl == 0) {
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int j = 0; j < NC; ++j) red[m * W + lane * NC + j] = acc[m][j];
    }
    sk_cluster_sync();
    if (rank == 0 && kl == 0 && live) {
        for (uint32_t r = 1; r < cs; ++r) {
#pragma unroll
            for (int m = 0; m < MT; ++m)
#pragma unroll
                for (int j = 0; j < NC; ++j) acc[m][j] += sk_ld_remote(&red[m * W + lane * NC + j], r);
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m < p.M) {
                Pack<T, NC> o;
#pragma unroll
                for (int j = 0; j < NC; ++j) o.v[j] = from_compute<T>(compute_t<T>(acc[m][j]));
                *reinterpret_cast<Pack<T, NC> *>(C + int64_t(m) * p.N + n0) = o;
            }
        }
    }
    sk_cluster_sync();  // nobody leaves while rank 0 may still read its shared memory
}

template <typename T, int MT, int NC>
int launch_skinny_t(const T *A, const T *B, T *C, int64_t batch, int M, int N, int K, cudaStream_t st) {
    constexpr int W = 32 * NC;
    const int strips = (N + W - 1) / W;
    // enough CTAs for ~2 per SM, at most 8 per cluster, and slices of at least 64 rows
    int cs = 1;
    while (cs < 8 && strips * cs * int(batch) < 2 * sm_count() && K / (cs * 2) >= 64) cs *= 2;
    int kchunk = (K + cs - 1) / cs;
    kchunk = (kchunk + SK_KL - 1) / SK_KL * SK_KL;
    const size_t smem = size_t(SK_KL / 2) * MT * W * sizeof(float) + size_t(MT) * kchunk * sizeof(T);
    if (smem > 200 * 1024) return DX_E_UNSUPPORTED;  // A's slice does not fit: the caller takes another path
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] {
        attr_err = cudaFuncSetAttribute(gemm_skinny_kernel<T, MT, NC>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    });
    if (attr_err != cudaSuccess) return fail(DX_E_CUDA, "matmul(skinny): cudaFuncSetAttribute: %s", cudaGetErrorString(attr_err));
    SkinnyParams p{M, N, K, kchunk};
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(strips * cs), unsigned(batch), 1);
    cfg.blockDim = dim3(SK_THREADS, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = unsigned(cs);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_skinny_kernel<T, MT, NC>, A, B, C, p);
    if (e != cudaSuccess) return fail(DX_E_CUDA, "matmul(skinny): %s", cudaGetErrorString(e));
    return check_launch("matmul(skinny)");
}

template <typename T> int launch_skinny(const T *A, const T *B, T *C, int64_t batch, int M, int N, int K, cudaStream_t st) {
    constexpr int V = 16 / int(sizeof(T));  // elements per 16-byte load
    if (M <= 1) return launch_skinny_t<T, 1, V>(A, B, C, batch, M, N, K, st);
    if (M <= 2) return launch_skinny_t<T, 2, V>(A, B, C, batch, M, N, K, st);
    if (M <= 4) return launch_skinny_t<T, 4, V>(A, B, C, batch, M, N, K, st);
    if (M <= 8) return launch_skinny_t<T, 8, V>(A, B, C, batch, M, N, K, st);
    return launch_skinny_t<T, 16, V / 2>(A, B, C, batch, M, N, K, st);  // 16 rows: half-width loads keep the accumulators in registers
}

}  // namespace

// Called by dx_matmul.  DX_E_UNSUPPORTED = not a shape for this kernel (the caller goes on).
int matmul_skinny(int dtype, const void *A, const void *B, void *C, int64_t batch, int64_t M, int64_t N, int64_t K, cudaStream_t st) {
    if (M > 16 || batch > 65535 || K < 8) return DX_E_UNSUPPORTED;
    const int es = dx_dtype_size(dtype);
    if (es != 2 && es != 4) return DX_E_UNSUPPORTED;
    // Each element of B costs M multiply-adds on the FMA pipe here, so the kernel stays bound by memory
    // only for very few rows: beyond that the tensor-core tile kernels are faster even at 1/8 occupancy
    // of their tiles (measured: 16-bit 2 rows, float32 8 rows; DX_GEMM_SKINNY_ROWS overrides).
    const char *env_rows = std::getenv("DX_GEMM_SKINNY_ROWS");
    const int forced_rows = env_rows ? std::atoi(env_rows) : 0;
    const int max_rows = forced_rows > 0 ? forced_rows : (es == 2 ? 2 : 8);
    if (M > max_rows) return DX_E_UNSUPPORTED;
    if (N % (16 / es) != 0 || !aligned_to(B, 16) || !aligned_to(C, 16)) return DX_E_UNSUPPORTED;
    switch (dtype) {
        case DX_BF16: return launch_skinny<bf16>((const bf16 *)A, (const bf16 *)B, (bf16 *)C, batch, int(M), int(N), int(K), st);
        case DX_F16: return launch_skinny<f16>((const f16 *)A, (const f16 *)B, (f16 *)C, batch, int(M), int(N), int(K), st);
        case DX_F32: return launch_skinny<float>((const float *)A, (const float *)B, (float *)C, batch, int(M), int(N), int(K), st);
        default: return DX_E_UNSUPPORTED;
    }
}

}  // namespace dx
