// C entry points of the EXL3 linear: host validation in berth's order and wording, then the
// fused decode GEMV (size_m <= 32 per launch).
#include "common.cuh"
#include "../../include/berth_b200.h"

#include <algorithm>
#include <cstring>

namespace berth {

std::string launch_gemm_tc(const void* a, const void* trellis, void* c, const void* suh, void* a_had, const void* svh,
                           int size_m, int size_k, int size_n, int k_bits, int codebook, int out_fp32, unsigned* status,
                           cudaStream_t stream);

std::string launch_gemm_tc_splitk(const void* a, const void* trellis, void* c, const void* suh, void* a_had, const void* svh,
                                  int size_m, int size_k, int size_n, int k_bits, int codebook, int out_fp32, const GemvScratch& sc,
                                  int sms, cudaStream_t stream);

// Where the persistent split-K tensor-core kernel takes over from the decode GEMV (measured on the 27B shapes at 4 and
// 6 bpw): from 17 rows -- the GEMV's third and fourth row group cost it 5 us on a 45 MB matrix, the tensor-core kernel's
// time does not depend on the row count -- and only for matrices with at least eight 64 x 128 weight stages per SM; below
// that its three launches (rotation, main kernel, finishing kernel) cost more than they save.
constexpr int kSplitKMinRows = 17;
constexpr long long kSplitKMinStagesPerSm = 8;

// Three kernels serve every row count: the fused decode GEMV up to 16 rows (and for small matrices up to 32), the
// persistent split-K tensor-core kernel for 17..32 rows, the tiled tensor-core GEMM above.
std::string linear_rows(const void* a, const void* trellis, void* c, const void* suh, void* a_had, const void* svh,
                        int size_m, int size_k, int size_n, int k_bits, int codebook, int out_fp32, cudaStream_t stream)
{
    const int device = current_device();
    const DeviceInfo& info = device_info(device);
    if (info.major != 10)
        throw std::runtime_error("exl3 linear: no linked kernel for this GPU (library is built for sm_100a only)");
    GemvScratch w = gemv_workspace(device);
    const long long stages = (long long) (size_n / 128) * (size_k / 64);
    if (size_m < kSplitKMinRows || (size_m <= 32 && stages < kSplitKMinStagesPerSm * info.sms))
        return launch_gemv(a, trellis, c, suh, a_had, svh, size_m, size_k, size_n, k_bits, codebook, out_fp32, w, info.sms,
                           stream);
    if (size_m <= 32)
        return launch_gemm_tc_splitk(a, trellis, c, suh, a_had, svh, size_m, size_k, size_n, k_bits, codebook, out_fp32, w,
                                     info.sms, stream);
    return launch_gemm_tc(a, trellis, c, suh, a_had, svh, size_m, size_k, size_n, k_bits, codebook, out_fp32, w.status, stream);
}

namespace {

// Checks of crates/berth-kernels/csrc/linear.cu:224-237 (berth), same order, same wording.
void check_linear_args(const char* who, const void* a, const void* trellis, const void* c, const void* suh,
                       const void* a_had, const void* svh, int size_k, int size_n, int k_bits, int codebook)
{
    const std::string w(who);
    if (!a || !trellis || !c || !suh || !a_had || !svh) throw std::runtime_error(w + ": null device pointer");
    if (size_k < 1 || size_n < 1) throw std::runtime_error(w + ": sizes must be positive");
    if (k_bits < 1 || k_bits > 8) throw std::runtime_error(w + ": K must be in 1..=8");
    if (codebook < 0 || codebook > 2) throw std::runtime_error(w + ": codebook must be 0 (default), 1 (mcg), or 2 (mul1)");
    if (size_k % 16 != 0) throw std::runtime_error(w + ": size_k must be a multiple of 16");
    if (size_n % 128 != 0) throw std::runtime_error(w + ": size_n must be a multiple of 128");
}

struct DevBuf {
    void* p = nullptr;
    ~DevBuf() { if (p) cudaFree(p); }
    void* alloc(size_t bytes)
    {
        cuda_ok(cudaMalloc(&p, bytes), "smoke cudaMalloc");
        cuda_ok(cudaMemset(p, 0, bytes), "smoke cudaMemset");
        return p;
    }
};

int smoke(int m, int k, int n, int bits, int cb, int out_fp32)
{
    CallState& st = exl3_state();
    try {
        DevBuf a, t, c, suh, ah, svh;
        size_t tb = size_t(k / 16) * (n / 16) * 16 * bits * 2;
        int rc = berth_exl3_linear(a.alloc(size_t(m) * k * 2), t.alloc(tb), c.alloc(size_t(m) * n * (out_fp32 ? 4 : 2)),
                                   suh.alloc(size_t(k) * 2), ah.alloc(size_t(m) * k * 2), svh.alloc(size_t(n) * 2), m, k,
                                   n, bits, cb, out_fp32, nullptr);
        if (rc != 0) return rc;
        cuda_ok(cudaDeviceSynchronize(), "smoke sync");
        return 0;
    } catch (const std::exception& e) {
        st.err = e.what();
        cudaGetLastError();
        return -1;
    }
}

}  // namespace
}  // namespace berth

using namespace berth;

extern "C" int berth_exl3_linear(const void* a, const void* trellis, void* c, const void* suh, void* a_had,
                                 const void* svh, int size_m, int size_k, int size_n, int k_bits, int codebook,
                                 int out_fp32, void* stream)
{
    CallState& st = exl3_state();
    return guarded(st, [&] {
        if (!a || !trellis || !c || !suh || !a_had || !svh) throw std::runtime_error("exl3 linear: null device pointer");
        if (size_m < 1 || size_k < 1 || size_n < 1) throw std::runtime_error("exl3 linear: sizes must be positive");
        check_linear_args("exl3 linear", a, trellis, c, suh, a_had, svh, size_k, size_n, k_bits, codebook);
        st.launch = linear_rows(a, trellis, c, suh, a_had, svh, size_m, size_k, size_n, k_bits, codebook, out_fp32,
                                (cudaStream_t) stream);
    });
}

// The decode linear with the greedy arg-max of every output row taken in the finishing step (an lm_head whose
// logits need not be written): berth runs the linear and then its two-kernel fused sampler over the logits
// (crates/berth-kernels/csrc/linear.cu:131-207 for the K = 6 head, csrc/sample/fused.cu:45-135 mode 0).
extern "C" int berth_exl3_linear_argmax(const void* a, const void* trellis, void* c, const void* suh, void* a_had,
                                        const void* svh, unsigned long long* best, int size_m, int size_k, int size_n,
                                        int k_bits, int codebook, int out_fp32, void* stream)
{
    CallState& st = exl3_state();
    return guarded(st, [&] {
        if (!a || !trellis || !suh || !a_had || !svh || !best) throw std::runtime_error("exl3 linear argmax: null device pointer");
        if (size_m < 1 || size_k < 1 || size_n < 1) throw std::runtime_error("exl3 linear argmax: sizes must be positive");
        if (size_m > 32) throw std::runtime_error("exl3 linear argmax: size_m must be <= 32 (the decode kernel)");
        check_linear_args("exl3 linear argmax", a, trellis, best, suh, a_had, svh, size_k, size_n, k_bits, codebook);
        const int device = current_device();
        const DeviceInfo& info = device_info(device);
        if (info.major != 10)
            throw std::runtime_error("exl3 linear argmax: no linked kernel for this GPU (library is built for sm_100a only)");
        cuda_ok(cudaMemsetAsync(best, 0, size_t(size_m) * sizeof(unsigned long long), (cudaStream_t) stream), "argmax keys memset");
        st.launch = launch_gemv(a, trellis, c, suh, a_had, svh, size_m, size_k, size_n, k_bits, codebook, out_fp32,
                                gemv_workspace(device), info.sms, (cudaStream_t) stream, best) + " [arg-max in the finishing step]";
    });
}

// For hosts that write weights on the same stream directly before using them (streaming experts or layers in): after
// berth_exl3_weights_streamed(1) the decode kernels of this process fetch no weights before their predecessor on the
// stream has ended, which is berth's own ownership rule (crates/berth-kernels/src/lib.rs:126-133: stream order is
// enough); the default keeps the prefetch and asks the caller to have the weights final one kernel earlier.
namespace berth { int set_weights_streamed(int on); }
extern "C" int berth_exl3_weights_streamed(int on) { return berth::set_weights_streamed(on); }

// The same with the token drawn instead of the arg-max: berth's fused sampler in its second mode (Gumbel arg-max over
// logits * inv_temp, crates/berth-kernels/csrc/sample/fused.cu:45-135 mode 1) taken in the finishing step of the linear.
// mode 0 = greedy (berth_exl3_linear_argmax), 1 = Gumbel with the noise of (random, row, column).
extern "C" int berth_exl3_linear_sample(const void* a, const void* trellis, void* c, const void* suh, void* a_had,
                                        const void* svh, unsigned long long* best, int size_m, int size_k, int size_n,
                                        int k_bits, int codebook, int out_fp32, float inv_temp, unsigned int random, int mode,
                                        void* stream)
{
    CallState& st = exl3_state();
    return guarded(st, [&] {
        if (!a || !trellis || !suh || !a_had || !svh || !best) throw std::runtime_error("exl3 linear sample: null device pointer");
        if (size_m < 1 || size_k < 1 || size_n < 1) throw std::runtime_error("exl3 linear sample: sizes must be positive");
        if (size_m > 32) throw std::runtime_error("exl3 linear sample: size_m must be <= 32 (the decode kernel)");
        if (mode != 0 && mode != 1) throw std::runtime_error("exl3 linear sample: mode must be 0 or 1");
        if (!(inv_temp > 0.0f) || !(inv_temp < 3.0e38f)) throw std::runtime_error("exl3 linear sample: inv_temp must be positive and finite");
        check_linear_args("exl3 linear sample", a, trellis, best, suh, a_had, svh, size_k, size_n, k_bits, codebook);
        const int device = current_device();
        const DeviceInfo& info = device_info(device);
        if (info.major != 10)
            throw std::runtime_error("exl3 linear sample: no linked kernel for this GPU (library is built for sm_100a only)");
        SampleArgs sample;
        sample.inv_temp = inv_temp; sample.random = random; sample.gumbel = mode;
        cuda_ok(cudaMemsetAsync(best, 0, size_t(size_m) * sizeof(unsigned long long), (cudaStream_t) stream), "sample keys memset");
        st.launch = launch_gemv(a, trellis, c, suh, a_had, svh, size_m, size_k, size_n, k_bits, codebook, out_fp32,
                                gemv_workspace(device), info.sms, (cudaStream_t) stream, best, nullptr, sample) +
                    (mode ? " [Gumbel arg-max in the finishing step]" : " [arg-max in the finishing step]");
    });
}

// A stack of equally shaped MUL1 matrices applied to the same rows in one launch (gate and up of an MLP stored
// one behind the other): the units of all matrices share one persistent decode launch, so launch latency, pipeline
// ramp and the finishing kernel are paid once.
extern "C" int berth_exl3_linear_stack(const void* a, const void* trellis_stack, void* c, const void* suh_stack, void* a_had,
                                       const void* svh_stack, int n_matrices, int size_m, int size_k, int size_n, int k_bits,
                                       int codebook, int out_fp32, void* stream)
{
    CallState& st = exl3_state();
    return guarded(st, [&] {
        if (!a || !trellis_stack || !c || !suh_stack || !a_had || !svh_stack) throw std::runtime_error("exl3 linear stack: null device pointer");
        if (size_m < 1 || size_k < 1 || size_n < 1) throw std::runtime_error("exl3 linear stack: sizes must be positive");
        if (n_matrices < 1 || n_matrices > 16) throw std::runtime_error("exl3 linear stack: n_matrices must be in 1..=16");
        check_linear_args("exl3 linear stack", a, trellis_stack, c, suh_stack, a_had, svh_stack, size_k, size_n, k_bits, codebook);
        if (codebook != 2 || size_m > kI8MaxRows)
            throw std::runtime_error("exl3 linear stack: no linked kernel (MUL1 codebook and size_m <= 8 only)");
        const int device = current_device();
        const DeviceInfo& info = device_info(device);
        if (info.major != 10)
            throw std::runtime_error("exl3 linear stack: no linked kernel for this GPU (library is built for sm_100a only)");
        st.launch = launch_gemv_i8(a, trellis_stack, c, suh_stack, a_had, svh_stack, size_m, size_k, size_n, k_bits, out_fp32,
                                   gemv_workspace(device), info.sms, (cudaStream_t) stream, nullptr, n_matrices);
    });
}

// Up to four MUL1 matrices of different widths applied to the same rows in one decode launch (q, k and v of an attention
// block): what berth does with one berth_ops_mgemm call over column slices (crates/berth-kernels/src/ops.rs:257-262), with
// the pointer lists in HOST memory, so that the library can encode one TMA view per matrix and rotate inside the kernel.
extern "C" int berth_exl3_linear_multi(const void* a, const void* const* trellis_list, void* const* c_list,
                                       const void* const* suh_list, void* const* a_had_list, const void* const* svh_list,
                                       const int* size_n_list, int n_matrices, int size_m, int size_k, int k_bits, int codebook,
                                       int out_fp32, void* stream)
{
    CallState& st = exl3_state();
    return guarded(st, [&] {
        if (!a || !trellis_list || !c_list || !suh_list || !a_had_list || !svh_list || !size_n_list)
            throw std::runtime_error("exl3 linear multi: null pointer");
        if (n_matrices < 1 || n_matrices > 4) throw std::runtime_error("exl3 linear multi: n_matrices must be in 1..=4");
        if (size_m < 1 || size_k < 1) throw std::runtime_error("exl3 linear multi: sizes must be positive");
        for (int i = 0; i < n_matrices; ++i) {
            if (size_n_list[i] < 1) throw std::runtime_error("exl3 linear multi: sizes must be positive");
            check_linear_args("exl3 linear multi", a, trellis_list[i], c_list[i], suh_list[i], a_had_list[i], svh_list[i], size_k,
                              size_n_list[i], k_bits, codebook);
        }
        if (codebook != 2 || size_m > kI8MaxRows)
            throw std::runtime_error("exl3 linear multi: no linked kernel (MUL1 codebook and size_m <= 8 only)");
        const int device = current_device();
        const DeviceInfo& info = device_info(device);
        if (info.major != 10)
            throw std::runtime_error("exl3 linear multi: no linked kernel for this GPU (library is built for sm_100a only)");
        st.launch = launch_gemv_i8_multi(a, trellis_list, c_list, suh_list, a_had_list, svh_list, size_n_list, n_matrices, size_m,
                                         size_k, k_bits, out_fp32, gemv_workspace(device), info.sms, (cudaStream_t) stream);
    });
}

// The decode linear with the residual added in its last step: c = residual + linear(a), fp32, size_m <= 32.  What berth
// does with berth_exl3_linear followed by berth_ops_add_f32 (crates/berth-engine/src/model.rs:976-1022: x = x + mlp(h2)).
extern "C" int berth_exl3_linear_add(const void* a, const void* trellis, void* c, const void* suh, void* a_had, const void* svh,
                                     const void* residual, int size_m, int size_k, int size_n, int k_bits, int codebook, void* stream)
{
    CallState& st = exl3_state();
    return guarded(st, [&] {
        if (!a || !trellis || !c || !suh || !a_had || !svh || !residual) throw std::runtime_error("exl3 linear add: null device pointer");
        if (size_m < 1 || size_k < 1 || size_n < 1) throw std::runtime_error("exl3 linear add: sizes must be positive");
        if (size_m > 32) throw std::runtime_error("exl3 linear add: size_m must be <= 32 (the decode kernels)");
        check_linear_args("exl3 linear add", a, trellis, c, suh, a_had, svh, size_k, size_n, k_bits, codebook);
        const int device = current_device();
        const DeviceInfo& info = device_info(device);
        if (info.major != 10)
            throw std::runtime_error("exl3 linear add: no linked kernel for this GPU (library is built for sm_100a only)");
        st.launch = launch_gemv(a, trellis, c, suh, a_had, svh, size_m, size_k, size_n, k_bits, codebook, 1, gemv_workspace(device), info.sms,
                                (cudaStream_t) stream, nullptr, static_cast<const float*>(residual)) + " [residual added in the last step]";
    });
}

// The down projection of an MLP with the activation taken on the fly: c = [residual +] linear(silu(gate) * up).  What berth
// does with berth_ops_silu_mul, berth_exl3_linear and (in the decode block) berth_ops_add_f32
// (crates/berth-engine/src/mlp.rs:128-160, model.rs:976-1022), without the launch and the buffer of the activation.
extern "C" int berth_exl3_linear_silu(const void* gate, const void* up, const void* trellis, void* c, const void* suh, void* a_had,
                                      const void* svh, const void* residual, float act_limit, int size_m, int size_k, int size_n,
                                      int k_bits, int codebook, int out_fp32, void* stream)
{
    CallState& st = exl3_state();
    return guarded(st, [&] {
        if (!gate || !up || !trellis || !c || !suh || !a_had || !svh) throw std::runtime_error("exl3 linear silu: null device pointer");
        if (size_m < 1 || size_k < 1 || size_n < 1) throw std::runtime_error("exl3 linear silu: sizes must be positive");
        if (size_m > 32) throw std::runtime_error("exl3 linear silu: size_m must be <= 32 (the decode kernels)");
        if (residual && !out_fp32) throw std::runtime_error("exl3 linear silu: the residual is added to fp32 outputs only");
        check_linear_args("exl3 linear silu", gate, trellis, c, suh, a_had, svh, size_k, size_n, k_bits, codebook);
        const int device = current_device();
        const DeviceInfo& info = device_info(device);
        if (info.major != 10)
            throw std::runtime_error("exl3 linear silu: no linked kernel for this GPU (library is built for sm_100a only)");
        ActInput act;
        act.up = up;
        act.limit = act_limit;
        st.launch = launch_gemv(gate, trellis, c, suh, a_had, svh, size_m, size_k, size_n, k_bits, codebook, out_fp32,
                                gemv_workspace(device), info.sms, (cudaStream_t) stream, nullptr, static_cast<const float*>(residual),
                                SampleArgs{}, act) + " [silu(gate) * up in the rotation" + (residual ? ", residual added in the last step]" : "]");
    });
}

extern "C" void berth_argmax_key_decode(unsigned long long key, int32_t* token, float* value)
{
    const uint32_t ord = uint32_t(key >> 32);
    const uint32_t bits = (ord & 0x80000000u) ? (ord & 0x7fffffffu) : ~ord;
    if (token) *token = int32_t(0xffffffffu - uint32_t(key & 0xffffffffu));
    if (value) std::memcpy(value, &bits, 4);
}

extern "C" int berth_prefill_exl3_linear(const void* a, const void* trellis, void* c, const void* suh, void* a_had,
                                         const void* svh, void* w_scratch, int size_m, int size_k, int size_n,
                                         int k_bits, int codebook, int c_fp32, void* stream)
{
    CallState& st = prefill_state();
    return guarded(st, [&] {
        // crates/berth-kernels/csrc/prefill_lin/linear.cu:248-266 (berth)
        if (!a || !trellis || !c || !suh || !a_had || !svh)
            throw std::runtime_error("prefill exl3 linear: null device pointer");
        if (size_m < 2) throw std::runtime_error("prefill exl3 linear: size_m must be > 1 (m = 1 is exl3_linear)");
        check_linear_args("prefill exl3 linear", a, trellis, c, suh, a_had, svh, size_k, size_n, k_bits, codebook);
        if (size_m > 144 && !w_scratch)
            throw std::runtime_error(
                "prefill exl3 linear: w_scratch (fp16, size_k * min(size_n, 32768)) is required when rows > 144");
        st.launch = linear_rows(a, trellis, c, suh, a_had, svh, size_m, size_k, size_n, k_bits, codebook, c_fp32,
                                (cudaStream_t) stream);
    });
}

// Smallest shapes of the two regimes berth's self tests exercise (csrc/linear.cu:406-465 of berth-kernels).
extern "C" int berth_exl3_smoke_int8(int out_fp32) { return smoke(1, 128, 256, 4, 2, out_fp32); }
extern "C" int berth_exl3_smoke_gemm(void) { return smoke(1, 128, 512, 6, 2, 0); }

// ------------------------------------------------------------------------------------------
// Sliced multi-linear (crates/berth-kernels/src/ops.rs:247-367, csrc/ops/mgemm.cu:125-334 of berth): several
// column slices of several trellis matrices applied to one input in one decode launch.  Host checks in
// berth's order and wording; every K and codebook is linked here, only the sliced mode is.
namespace berth {
std::string launch_gemv_sliced(const void* a, const void* b_list, const void* suh_list, void* a_had, const void* svh_list,
                               const void* c_list, const int* n_stride_list, const int* had_src_list, int num_had_src, int n_slices,
                               int size_m, int size_k, int size_n, int k_bits, int codebook, int out_fp32, const GemvScratch& sc,
                               int sms, cudaStream_t stream, long long a_src_stride = 0);
std::string launch_gemv_uniform(const void* a, const void* b_list, const void* suh_list, void* a_had, const void* svh_list, void* c,
                                int count, bool per_matrix_input, int size_m, int size_k, int size_n, int k_bits, int codebook,
                                int out_fp32, const GemvScratch& sc, int sms, cudaStream_t stream);
}

extern "C" int berth_ops_mgemm(const void* a, const void* b_list, void* c, const void* suh_list, void* a_had, const void* svh_list,
                               int size_m, int size_k, int size_n, int k_bits, int codebook, int c_fp32, int bszm_in, int bszm_out,
                               const int* size_n_list, const void* c_ptrs, const int* n_stride_list, const int* had_src_list,
                               int num_had_src, void* stream)
{
    using namespace berth;
    CallState& st = ops_state();
    int tag = 0;
    const int rc = guarded(st, [&] {
        if (!a || !b_list || !c || !suh_list || !a_had || !svh_list) throw std::runtime_error("exl3_mgemm: null device pointer");
        if (size_m < 1 || size_k < 1 || size_n < 1 || bszm_in < 1 || bszm_out < 1)
            throw std::runtime_error("exl3_mgemm: sizes must be positive");
        if (size_k % 16 != 0) throw std::runtime_error("exl3_mgemm: size_k must be a multiple of 16");
        if (size_n % 128 != 0) throw std::runtime_error("exl3_mgemm: size_n must be a multiple of 128");
        if (k_bits < 1 || k_bits > 8 || codebook < 0 || codebook > 2)
            throw std::runtime_error("exl3_mgemm: no linked kernel for K=" + std::to_string(k_bits) + " codebook=" + std::to_string(codebook));
        if (c_fp32 != 0 && c_fp32 != 1) throw std::runtime_error("exl3_mgemm: c_fp32 must be 0 (fp16) or 1 (fp32)");
        const bool any_list = size_n_list || c_ptrs || n_stride_list || had_src_list;
        if (any_list) {
            if (!size_n_list || !c_ptrs || !n_stride_list || !had_src_list)
                throw std::runtime_error("exl3_mgemm: sliced mode requires size_n_list, c_ptrs, n_stride_list, and had_src_list");
            if (num_had_src < 1) throw std::runtime_error("exl3_mgemm: sliced mode needs one suh entry per source");
            if (bszm_in != 1) throw std::runtime_error("exl3_mgemm: sliced mode is single-input");
        } else {
            // uniform mode: bszm_out equally shaped matrices, outputs (bszm_out, size_m, size_n), one input for all or one each
            if (num_had_src != 0) throw std::runtime_error("exl3_mgemm: num_had_src requires had_src_list");
            if (bszm_in != 1 && bszm_in != bszm_out)
                throw std::runtime_error("exl3_mgemm: uniform mode takes one input for all matrices or one per matrix (bszm_in = 1 or bszm_out)");
        }
        const int device = current_device();
        const DeviceInfo& info = device_info(device);
        if (info.major != 10) throw std::runtime_error("exl3_mgemm: no linked kernel for this GPU (library is built for sm_100a only)");
        if (!any_list)
            st.launch = launch_gemv_uniform(a, b_list, suh_list, a_had, svh_list, c, bszm_out, bszm_in > 1, size_m, size_k, size_n, k_bits,
                                            codebook, c_fp32, gemv_workspace(device), info.sms, (cudaStream_t) stream);
        else
        st.launch = launch_gemv_sliced(a, b_list, suh_list, a_had, svh_list, c_ptrs, n_stride_list, had_src_list, num_had_src, bszm_out,
                                       size_m, size_k, size_n, k_bits, codebook, c_fp32, gemv_workspace(device), info.sms,
                                       (cudaStream_t) stream);
        tag = size_m <= 8 ? 1 : (size_m <= 16 ? 2 : 4);   // the token groups of the launch, as the positive "shape tag"
    });
    return rc == 0 ? tag : rc;
}
