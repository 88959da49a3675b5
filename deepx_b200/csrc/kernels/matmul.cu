// dx_matmul placeholder until the tcgen05 kernel lands.
#include "common.cuh"
extern "C" int dx_matmul(int dtype, const void *A, const void *B, void *C, int64_t batch, int64_t M, int64_t N, int64_t K,
                         void *stream) {
    (void)A; (void)B; (void)C; (void)batch; (void)M; (void)N; (void)K; (void)stream;
    return dx::fail(DX_E_UNSUPPORTED, "matmul: not built yet (dtype code %d)", dtype);
}
