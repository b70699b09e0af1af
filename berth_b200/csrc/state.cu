// Host-side state of the library: per-thread status strings, per-device facts and the
// split-K workspace of the decode GEMV; plus the pure-integer entry points berth's tests pin.
#include "common.cuh"

#include <algorithm>
#include "../../include/berth_b200.h"

#include <atomic>
#include <mutex>

namespace berth {

int read_gemv_status(int device);

CallState& exl3_state()    { thread_local CallState s; return s; }
CallState& prefill_state() { thread_local CallState s; return s; }
CallState& ops_state()     { thread_local CallState s; return s; }
CallState& moe_state()     { thread_local CallState s; return s; }

namespace {
std::mutex g_mu;
DeviceInfo g_info[kMaxDevices];
GemvScratch g_ws[kMaxDevices];
}  // namespace

int current_device()
{
    int device = 0;
    cuda_ok(cudaGetDevice(&device), "cudaGetDevice");
    if (device < 0 || device >= kMaxDevices) throw std::runtime_error("device index out of range");
    return device;
}

const DeviceInfo& device_info(int device)
{
    std::lock_guard<std::mutex> lock(g_mu);
    if (device < 0 || device >= kMaxDevices) throw std::runtime_error("device index out of range");
    DeviceInfo& d = g_info[device];
    if (!d.sms) {
        int major = 0, minor = 0, sms = 0;
        cuda_ok(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device), "compute capability");
        cuda_ok(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device), "compute capability");
        cuda_ok(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device), "multiProcessorCount");
        // Classes in the order of the fork's CC_* constants (crates/berth-kernels/csrc/linear.cu:310-319).
        int cc = 1;
        if (major >= 10) cc = 5;
        else if (major >= 9) cc = 4;
        else if (major >= 8 && minor >= 9) cc = 3;
        else if (major >= 8) cc = 2;
        d.cc = cc;
        d.major = major;
        d.sms = sms;
    }
    return d;
}

namespace { std::atomic<int> g_weights_streamed{0}; }
bool weights_streamed() { return g_weights_streamed.load(std::memory_order_relaxed) != 0; }
int set_weights_streamed(int on) { return g_weights_streamed.exchange(on ? 1 : 0); }

GemvScratch gemv_workspace(int device)
{
    std::lock_guard<std::mutex> lock(g_mu);
    if (device < 0 || device >= kMaxDevices) throw std::runtime_error("device index out of range");
    GemvScratch& w = g_ws[device];
    if (!w.slabs) {
        const size_t blocksum = kGemvBlocksumFloats * sizeof(float);
        const size_t total = kGemvSlabBytes + kGemvAfragBytes + blocksum + kGemvCounterWords * sizeof(unsigned) + kGemvListEntries * 16 + 256;
        void* p = nullptr;
        cuda_ok(cudaMalloc(&p, total), "gemv workspace");
        cuda_ok(cudaMemset(p, 0, total), "gemv workspace memset");
        char* b = static_cast<char*>(p);
        w.slabs = reinterpret_cast<float*>(b);
        w.slab_bytes = kGemvSlabBytes;
        b += kGemvSlabBytes;
        w.afrag = reinterpret_cast<uint32_t*>(b);
        w.afrag_bytes = kGemvAfragBytes;
        b += kGemvAfragBytes;
        w.blocksum = reinterpret_cast<float*>(b);
        w.blocksum_floats = kGemvBlocksumFloats;
        b += blocksum;
        w.counters = reinterpret_cast<unsigned*>(b);
        w.counter_words = kGemvCounterWords;
        b += kGemvCounterWords * sizeof(unsigned);
        w.lists = reinterpret_cast<unsigned long long*>(b);
        b += kGemvListEntries * 16;
        w.status = reinterpret_cast<unsigned*>(b);
    }
    return w;
}

// Reads and clears the status word of the library's scratch on `device` (synchronises).
// 0 = every bounded wait of the decode kernels completed.
int read_static_status(int device);   // gemv.cu: the fixed in-image scratch of the allocation-free entry point

int read_gemv_status(int device)
{
    GemvScratch w;
    {
        std::lock_guard<std::mutex> lock(g_mu);
        w = g_ws[device];
    }
    if (!w.status) return 0;
    unsigned v = 0;
    cuda_ok(cudaMemcpy(&v, w.status, sizeof v, cudaMemcpyDeviceToHost), "status read");
    if (v) cuda_ok(cudaMemset(w.status, 0, sizeof v), "status clear");
    return int(v);
}

}  // namespace berth

using namespace berth;

extern "C" int berth_device_cc(int device)
{
    try { return device_info(device).cc; } catch (const std::exception&) { cudaGetLastError(); return -1; }
}

extern "C" int berth_device_status(int device)
{
    try { return berth::read_gemv_status(device) | berth::read_static_status(device); } catch (const std::exception&) { cudaGetLastError(); return -1; }
}

extern "C" int berth_device_sms(int device)
{
    try { return device_info(device).sms; } catch (const std::exception&) { cudaGetLastError(); return -1; }
}

extern "C" const char* berth_exl3_last_error(void)     { return exl3_state().err.c_str(); }
extern "C" const char* berth_exl3_last_launch(void)    { return exl3_state().launch.c_str(); }
extern "C" const char* berth_prefill_last_error(void)  { return prefill_state().err.c_str(); }
extern "C" const char* berth_prefill_last_launch(void) { return prefill_state().launch.c_str(); }
extern "C" const char* berth_ops_last_error(void)      { return ops_state().err.c_str(); }
extern "C" const char* berth_ops_last_launch(void)     { return ops_state().launch.c_str(); }

// FNV-1a over the shape, m bucketed (csrc/linear.cu:65-104 of berth-kernels); m = 1 shares the m = 2 entry.
extern "C" uint64_t berth_exl3_gemm_tune_key(int size_m, int size_k, int size_n, int k_bits, int out_fp32,
                                             int device, int cc, int sms, int cb)
{
    int m = size_m < 2 ? 2 : size_m;
    uint64_t mk;
    if (m <= 16) { mk = 1; while (mk < (uint64_t) m) mk <<= 1; if (mk > 16) mk = 16; }
    else if (m <= 31) mk = 32;
    else if (m <= 63) mk = 64;
    else if (m <= 127) mk = 128;
    else mk = 512;
    uint64_t h = 1469598103934665603ull;
    const uint64_t v[9] = {mk, (uint64_t) size_k, (uint64_t) size_n, (uint64_t) k_bits, out_fp32 ? 1ull : 0ull,
                           (uint64_t) device, (uint64_t) cc, (uint64_t) sms, (uint64_t) cb};
    for (uint64_t x : v) { h ^= x; h *= 1099511628211ull; }
    return h;
}

// FNV-1a key of the fork's multi-linear autotune cache (csrc/ops/mgemm.cu:40-91,277-294 of berth-kernels):
// m bucketed to a power of two up to 16 (m = 1 stays 1), batch sizes capped at 24, sliced launches salted.
extern "C" uint64_t berth_ops_mgemm_tune_key(int size_m, int size_k, int size_n, int k_bits, int c_fp32, int device, int cc,
                                             int sms, int cb, int bszm_in, int bszm_out, int sliced)
{
    uint64_t mk;
    if (size_m <= 16) { mk = 1; while (mk < (uint64_t) std::max(size_m, 1)) mk <<= 1; if (mk > 16) mk = 16; }
    else if (size_m <= 31) mk = 32;
    else if (size_m <= 63) mk = 64;
    else if (size_m <= 127) mk = 128;
    else mk = 512;
    uint64_t h = 1469598103934665603ull;
    const uint64_t v[11] = {mk, (uint64_t) size_k, (uint64_t) size_n, (uint64_t) k_bits, c_fp32 ? 1ull : 0ull, (uint64_t) device,
                            (uint64_t) cc, (uint64_t) sms, (uint64_t) cb, (uint64_t) std::min(bszm_in, 24), (uint64_t) std::min(bszm_out, 24)};
    for (uint64_t x : v) { h ^= x; h *= 1099511628211ull; }
    if (sliced) h ^= 0x9e3779b97f4a7c15ull;
    return h;
}

// Eligibility table of the fork's narrow/wide small-m GEMV (csrc/prefill_lin/gemv.cu:72-101 of
// berth-kernels): -1 ineligible, 0 narrow, 1 wide.  Integer logic only.
extern "C" int berth_exl3_gemv_cfg(int cc, int size_m, int size_k, int size_n, int K, int cb, int mode,
                                   int narrow_coresident)
{
    constexpr int kAmpere = 2, kAda = 3, kMaxM = 8;
    if (mode == 0) return -1;
    if (K < 2 || K > 4) return -1;
    if (K != 4 && cb == 0) return -1;
    if (size_m > kMaxM) return -1;
    if (size_k % 128 || size_n % 128) return -1;
    if (mode == 2) return size_n <= 8192 ? 0 : 1;
    if (mode == 3) return 0;
    if (mode == 4) return 1;
    if (K == 2) return size_n <= 8192 ? 0 : 1;
    if (K == 3 && cc == kAda) return size_n <= 8192 ? 0 : 1;
    if (size_n / 32 <= narrow_coresident) return 0;
    if (size_k <= 2048 && size_n <= 8192) return 0;
    if (K == 3) return -1;
    if (size_n >= 8192 && size_k <= 4096) return 1;
    if (size_n >= 8192 && size_n <= 10240 && size_k <= 5120 && cc == kAmpere) return 1;
    return -1;
}
