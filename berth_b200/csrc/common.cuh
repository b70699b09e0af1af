// Shared host/device helpers of libberth_b200: error convention of the C boundary, per-device
// state, small fp16 utilities.  sm_100a only.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <stdexcept>
#include <string>

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ < 1000)
#error "libberth_b200 is written for sm_100a (B200) only"
#endif

namespace berth {

// Host-side CUDA check: the message goes back through the C ABI, nothing aborts
// (same convention as crates/berth-kernels/csrc/check.cuh:8-14 of berth).
inline void cuda_ok(cudaError_t err, const char* what)
{
    if (err == cudaSuccess) return;
    throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(err));
}

// Programmatic dependent launch: the kernel may become resident while its predecessor on the
// stream is still running (hiding its launch latency), so it must execute pdl_wait() before its
// first access to anything the predecessor may have written, and should call pdl_trigger() early
// to extend the same courtesy to its own successor.  A predecessor that never triggers (any foreign
// kernel) behaves as an ordinary stream dependency.
template <typename... KArgs, typename... Args>
inline void launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, const char* what,
                       Args&&... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cuda_ok(cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...), what);
}
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

// One family of entry points = one pair of thread-local strings (last error / last launch).
struct CallState {
    std::string err;
    std::string launch;
    void clear() { err.clear(); launch.clear(); }
};
CallState& exl3_state();     // berth_exl3_*
CallState& prefill_state();  // berth_prefill_*
CallState& ops_state();      // berth_ops_*
CallState& moe_state();      // berth_moe_*

// Runs `fn`, turning any exception into rc -1 + message, clearing the sticky CUDA error the
// way crates/berth-kernels/csrc/linear.cu:377-394 does.
template <typename F>
inline int guarded(CallState& st, F&& fn)
{
    try {
        st.clear();
        fn();
        return 0;
    } catch (const std::exception& e) {
        st.err = e.what();
        st.launch.clear();
        cudaGetLastError();
        return -1;
    }
}

constexpr int kMaxDevices = 64;

struct DeviceInfo {
    int sms = 0;
    int cc = 0;       // 1 old, 2 Ampere, 3 Ada, 4 Hopper, 5 Blackwell
    int major = 0;
};
const DeviceInfo& device_info(int device);
int current_device();

// Scratch of the decode GEMV: fp32 partial-sum slabs (two [m][BU*128] slabs per CTA), the rotated
// activations in fragment order, one fp32 sum per (row, 128 rotated inputs), and a status word
// that collects bounded-wait failures.
struct GemvScratch {
    float* slabs = nullptr;
    size_t slab_bytes = 0;
    uint32_t* afrag = nullptr;     // rotated activations in MMA fragment order
    size_t afrag_bytes = 0;
    float* blocksum = nullptr;
    size_t blocksum_floats = 0;
    unsigned* counters = nullptr;  // integer tensor path: arrival counters of the band groups (zero between launches)
    size_t counter_words = 0;
    unsigned long long* lists = nullptr;   // slice lists the library writes itself (uniform multi-linear): kGemvListEntries each of
                                           // output addresses (8 bytes), row strides and source indices (4 bytes)
    unsigned* status = nullptr;
};
// The library's own scratch: allocated once per device at first use, never grown, never freed
// (cf. crates/berth-kernels/csrc/int8_sq.cu:20-47 of berth).
constexpr size_t kGemvSlabBytes = size_t(32) << 20;
constexpr size_t kGemvBlocksumFloats = size_t(32) * 4096;
constexpr size_t kGemvCounterWords = size_t(1) << 16;
constexpr size_t kGemvListEntries = 2048;
constexpr size_t kGemvAfragBytes = size_t(8) << 20;   // size_k * ceil(size_m / 8) <= 524288
GemvScratch gemv_workspace(int device);

// One problem of a grouped decode launch: matrix `z` of a trellis stack applied to `rows` (at most
// 8*TG) consecutive rows starting at `row0` of the activation / output row arrays.
struct GemvProblem {
    int z, row0, rows, pad;
};

// Rotation of the rows of a grouped tensor-core launch (see rotate_rows_grouped).
struct RotateArgs {
    const __half* src;     // input rows [.][k]; the gate outputs in silu mode
    const __half* src_u;   // silu mode: the up outputs
    const int32_t* perm;   // gather mode: row r < n_perm reads src row perm[r] / div, later rows read src row r - n_perm
    int div, n_perm;
    const __half* suh_a;   // [n_matrices][k]
    const __half* suh_b;   // dual mode: second scale stack
    __half* out_a;         // [max_rows][k]
    __half* out_b;         // dual mode: second output
    const GemvProblem* problems;
    const int* n_problems;
    int chunk, k, max_problems, n_matrices, max_rows;
};
// out_a[row] = fp16(H128(x[row] * suh_a[matrix of the row]) / sqrt(128)) for every row the problem table covers
// (and out_b with suh_b when `dual`); x = src, or silu(src) * src_u when `silu`, or gathered rows of src when a.perm is set.
void rotate_rows_grouped(const RotateArgs& a, bool dual, bool silu, int sms, cudaStream_t stream);
// launch_gemm_tc_grouped without its rotation: `xr_had` already holds the rotated rows.
std::string launch_gemm_tc_grouped_rotated(const void* xr_had, const void* trellis_stack, int n_matrices, void* c, const void* svh_stack,
                                           const GemvProblem* problems, const int* n_problems, int max_problems, int max_rows, int nsub,
                                           int size_k, int size_n, int k_bits, int codebook, int out_fp32, unsigned* status, int sms,
                                           cudaStream_t stream);

// Grouped prefill launch over a stack of equally shaped matrices on the tensor cores: problem i applies
// matrix z_i to rows [row0_i, row0_i + rows_i) of xr, rows_i <= 128 * nsub; xr_had [max_rows][k] fp16
// receives the rotated rows.
std::string launch_gemm_tc_grouped(const void* xr, void* xr_had, const void* trellis_stack, int n_matrices, void* c,
                                   const void* suh_stack, const void* svh_stack, const GemvProblem* problems, const int* n_problems,
                                   int max_problems, int max_rows, int nsub, int size_k, int size_n, int k_bits, int codebook,
                                   int out_fp32, unsigned* status, int sms, cudaStream_t stream);

#ifdef __CUDACC__
// A problem-table entry with every field forced into range, so that a table the caller forgot to
// build (or built for another shape) yields wrong numbers, never a wild address.
__device__ __forceinline__ GemvProblem load_problem(const GemvProblem* table, int i, int n_matrices, int tok, int max_rows)
{
    GemvProblem pr = table[i];
    pr.z = min(max(pr.z, 0), n_matrices - 1);
    pr.rows = min(max(pr.rows, 0), tok);
    pr.row0 = min(max(pr.row0, 0), max(max_rows - pr.rows, 0));
    return pr;
}
#endif

// Rotation of the rows of a grouped decode launch into MMA-fragment order (see rotate_rows_frag).
struct RotateFragArgs {
    const __half* src;     // input rows [.][k]; the gate outputs in silu mode
    const __half* src_u;   // silu mode: the up outputs
    const int32_t* perm;   // gather mode: row r < n_perm reads src row perm[r] / div, later rows read src row r - n_perm
    int div, n_perm;
    const __half* suh_a;   // [n_matrices][k]
    const __half* suh_b;   // dual mode: second scale stack
    uint32_t* afrag_a;     // max_problems * (k/16) * (tok/8) * 64 words
    uint32_t* afrag_b;     // dual mode
    float* bsum_a;         // max_problems * tok * (k/128) floats
    float* bsum_b;         // dual mode
    const GemvProblem* problems;
    const int* n_problems;
    int tok, k, max_problems, n_matrices, max_rows;   // tok = rows per problem: 8, 16 or 32
    int pair;              // dual mode: 1 = the second output is problem (index + problem count) of afrag_a / bsum_a (doubled table)
};
void rotate_rows_frag(const RotateFragArgs& a, bool dual, bool silu, int sms, cudaStream_t stream);
// launch_gemv_grouped without its rotation: afrag / blocksum already hold the rotated rows.
std::string launch_gemv_grouped_rotated(const void* trellis_stack, int n_experts, void* c, const void* svh_stack,
                                        const GemvProblem* problems, const int* n_problems, int max_problems, int max_rows, int tg,
                                        const uint32_t* afrag, float* blocksum, int size_k, int size_n, int k_bits, int codebook,
                                        int out_fp32, const GemvScratch& scratch, int sms, cudaStream_t stream);

// Grouped decode launch over a stack of equally shaped matrices (the experts of an MoE layer):
// `problems` / `n_problems` live on the device (built by the dispatch kernels), xr fp16 [R][k] are
// the routed rows, c the outputs [R][n]; suh_stack [experts][k], svh_stack [experts][n].
// Table entries are clamped on the device to max_problems, n_experts and max_rows (the number of
// rows of xr / c).  afrag / blocksum scratch must hold max_problems * (k/16) * tg * 256 bytes and
// max_problems * 8 * tg * (k/128) floats.
std::string launch_gemv_grouped(const void* xr, const void* trellis_stack, int n_experts, void* c, const void* suh_stack,
                                const void* svh_stack, const GemvProblem* problems, const int* n_problems, int max_problems,
                                int max_rows, int tg, uint32_t* afrag, float* blocksum, int size_k, int size_n, int k_bits,
                                int codebook, int out_fp32, const GemvScratch& scratch, int sms, cudaStream_t stream);

// How the arg-max keys of a decode launch are scored: the stored output itself (greedy), or
// output * inv_temp + Gumbel noise drawn from a counter hash of (random, row, column) -- one draw of the softmax
// distribution at temperature 1 / inv_temp (the Gumbel-max trick).
// Process-wide switch set by berth_exl3_weights_streamed: true when a caller may write a trellis on the stream directly
// before the linear that reads it; the decode kernels then fetch no weights ahead of griddepcontrol.wait.
bool weights_streamed();

struct SampleArgs {
    float inv_temp = 1.0f;
    unsigned random = 0;
    int gumbel = 0;
};
// With `up` set the linear's input is silu(a) * up (both fp16 [m][k]), clamped to +-limit when that is not 0: the
// rotation applies it on the fly, rounded step by step as k_silu_mul rounds it.
struct ActInput {
    const void* up = nullptr;
    float limit = 0.f;
};
std::string launch_gemv(const void* a, const void* trellis, void* c, const void* suh, void* a_had, const void* svh,
                        int size_m, int size_k, int size_n, int k_bits, int codebook, int out_fp32,
                        const GemvScratch& scratch, int sms, cudaStream_t stream, unsigned long long* argmax = nullptr,
                        const float* residual = nullptr, const SampleArgs& sample = SampleArgs{}, const ActInput& act = ActInput{});

// The same linear for the MUL1 codebook on the integer tensor path (gemv_i8.cu), up to kI8MaxRows rows; launch_gemv
// forwards one to four rows to it (above, the limb tiles of the rows cost more L2 traffic than the fp16 path's
// fragments), berth_exl3_linear_stack up to eight.
constexpr int kI8MaxRows = 8;
std::string launch_gemv_i8(const void* a, const void* trellis, void* c, const void* suh, void* a_had, const void* svh,
                           int size_m, int size_k, int size_n, int k_bits, int out_fp32, const GemvScratch& scratch, int sms,
                           cudaStream_t stream, unsigned long long* argmax, int n_stack = 1, const float* residual = nullptr,
                           const SampleArgs& sample = SampleArgs{}, const ActInput& act = ActInput{});

// The integer-path decode kernel over up to four MUL1 matrices of different widths applied to the same rows (host arrays
// of device pointers and widths); same contract as launch_gemv per matrix.
std::string launch_gemv_i8_multi(const void* a, const void* const* trellis, void* const* c, const void* const* suh,
                                 void* const* a_had, const void* const* svh, const int* size_n, int n_matrices, int size_m,
                                 int size_k, int k_bits, int out_fp32, const GemvScratch& sc, int sms, cudaStream_t stream);
// True when launch_gemv_i8 would rotate the activations inside the decode kernel for this dense shape.
bool gemv_i8_rotates_in_kernel(int size_m, int size_k, int size_n, int k_bits, int sms);

constexpr float kRScale = 0.088388347648f;  // 1/sqrt(128), csrc/prefill_lin/reconstruct.cu:43-44

}  // namespace berth
