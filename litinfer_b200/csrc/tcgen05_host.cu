// Host side shared by the tcgen05 kernels: the driver entry point that encodes tensor maps
// (resolved at run time, so the library does not link against the driver), the status word the
// kernels raise when a bounded wait runs out, and the status query of the C interface.
#include "tcgen05.cuh"

namespace tc {

static EncodeTiledFn g_encode = nullptr;
static int* g_error_host = nullptr;       // mapped pinned memory: the kernels write, the host reads without a sync
static int* g_error_dev = nullptr;

int setup(EncodeTiledFn* encode, int** error_host, int** error_dev) {
    if (!g_encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
        if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn)
            return li_fail("tcgen05: the driver has no cuTensorMapEncodeTiled: %s", cudaGetErrorString(e));
        g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    if (!g_error_host) {
        cudaError_t e = cudaHostAlloc((void**)&g_error_host, 1024 * sizeof(int), cudaHostAllocMapped);      // [0]: the status word; the rest: progress marks of kernels that are asked to leave them
        if (e != cudaSuccess) return li_fail("tcgen05: cannot allocate the status word: %s", cudaGetErrorString(e));
        for (int i = 0; i < 1024; ++i) g_error_host[i] = 0;
        e = cudaHostGetDevicePointer((void**)&g_error_dev, g_error_host, 0);
        if (e != cudaSuccess) return li_fail("tcgen05: cannot map the status word: %s", cudaGetErrorString(e));
    }
    *encode = g_encode;
    *error_host = g_error_host;
    *error_dev = g_error_dev;
    return 0;
}

int make_map(CUtensorMap* map, const void* base, int rows, int cols, int box_rows) {
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return li_fail("tcgen05: cuTensorMapEncodeTiled failed with %d for a [%d, %d] tensor", (int)r, rows, cols);
    return 0;
}

// The general form: a row-major [rows, cols] bfloat16 matrix in boxes of box_rows x box_cols with the 32-, 64- or
// 128-byte swizzle (box_cols * 2 bytes must not exceed the swizzle width), zero fill outside.
int make_map_ex(CUtensorMap* map, const void* base, unsigned long long rows, unsigned long long cols, unsigned box_cols, unsigned box_rows,
                int swizzle_bytes) {
    LI_REQUIRE(g_encode != nullptr, "tcgen05: make_map_ex before setup");
    LI_REQUIRE(box_rows >= 1 && box_rows <= 256 && box_cols >= 8 && box_cols * 2 <= (unsigned)swizzle_bytes && (cols * 2) % 16 == 0,
               "tcgen05: bad tensor map (box %u x %u, swizzle %d, %llu columns)", box_rows, box_cols, swizzle_bytes, cols);
    const CUtensorMapSwizzle sw = swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                  : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return li_fail("tcgen05: cuTensorMapEncodeTiled failed with %d for a [%llu, %llu] tensor in boxes of %u x %u", (int)r, rows, cols, box_rows, box_cols);
    return 0;
}

}  // namespace tc

// 0 while no launch of a tcgen05 kernel has given up a wait; else which role did
// (products: 1 producer, 2 tensor-core issuer, 3 epilogue; attention: 11, 12, 13 likewise).  Meaningful after a synchronisation.
LI_EXPORT int li_tcgen05_status() {
    tc::EncodeTiledFn f;
    int *h = nullptr, *d = nullptr;
    if (tc::setup(&f, &h, &d)) return -1;
    return *h;
}

// Clears the status word (after a test made a wait run out; a real run-out means the results since are invalid).
LI_EXPORT void li_tcgen05_clear_status() {
    tc::EncodeTiledFn f;
    int *h = nullptr, *d = nullptr;
    if (tc::setup(&f, &h, &d) == 0) *h = 0;
}

namespace {
// One thread waits, with a short limit, on a barrier that nobody arrives on: the wait runs out, the thread raises the
// status word and returns.  Nothing is in flight and no tensor memory is held, so there is nothing to clean up.
__global__ void wait_runs_out_kernel(unsigned long long limit_ns, int* error_flag, int code) {
    __shared__ unsigned long long bar;
    if (threadIdx.x == 0) {
        tc::mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (!tc::mbar_wait(&bar, 0, limit_ns)) atomicExch(error_flag, code);
    }
}
}  // namespace

// For tests: exercises the path a bounded wait takes when its limit runs out (limit in microseconds, at most a second).
// Afterwards li_tcgen05_status() reads 99 until li_tcgen05_clear_status().
LI_EXPORT int li_tcgen05_wait_selftest(int limit_us, cudaStream_t stream) {
    LI_REQUIRE(limit_us >= 1 && limit_us <= 1000000, "tcgen05 wait self-test: limit of %d us is outside [1, 1000000]", limit_us);
    tc::EncodeTiledFn f;
    int *h = nullptr, *d = nullptr;
    if (int rc = tc::setup(&f, &h, &d)) return rc;
    wait_runs_out_kernel<<<1, 32, 0, stream>>>((unsigned long long)limit_us * 1000ull, d, 99);
    return li_check_launch("tcgen05 wait self-test");
}

// Progress marks (words 1..1023 of the mapped status area), for kernels launched with their debug flag: what each CTA
// reached last.  Readable while a kernel is still running.
LI_EXPORT int li_tcgen05_progress(int* out, int n) {
    tc::EncodeTiledFn f;
    int *h = nullptr, *d = nullptr;
    if (tc::setup(&f, &h, &d)) return -1;
    for (int i = 0; i < n && i < 1023; ++i) out[i] = h[1 + i];
    return 0;
}
