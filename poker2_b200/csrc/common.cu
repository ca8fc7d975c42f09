// Error plumbing and per-device constant tables.
#include "common.cuh"
#include "rank7.cuh"

#include <cstdarg>
#include <cstdio>
#include <mutex>

namespace p2b {

static thread_local char g_error[512] = "";

int set_error(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

const char* last_error() { return g_error; }

int check_cuda(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return P2B_OK;
    return set_error(P2B_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

constexpr int kMaxDevices = 64;
static ComboTable* g_combo[kMaxDevices] = {nullptr};
static RankLut* g_rank_lut[kMaxDevices] = {nullptr};
static int g_sms[kMaxDevices] = {0};
static std::mutex g_mu;

static int current_device() {
    int dev = 0;
    cudaGetDevice(&dev);
    return dev;
}

int ensure_tables() {
    const int dev = current_device();
    if (dev < 0 || dev >= kMaxDevices) return set_error(P2B_ERR_STATE, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_mu);
    if (g_combo[dev]) return P2B_OK;
    ComboTable host;
    int h = 0;
    for (int a = 0; a < P2B_NUM_CARDS; ++a)
        for (int b = a + 1; b < P2B_NUM_CARDS; ++b, ++h) {
            host.c1[h] = (uint8_t)a;
            host.c2[h] = (uint8_t)b;
        }
    ComboTable* d = nullptr;
    int rc = check_cuda(cudaMalloc(&d, sizeof(ComboTable)), "cudaMalloc(combo table)");
    if (rc) return rc;
    rc = check_cuda(cudaMemcpy(d, &host, sizeof(ComboTable), cudaMemcpyHostToDevice), "cudaMemcpy(combo table)");
    if (rc) {
        cudaFree(d);
        return rc;
    }
    static RankLut lut;  // 33 KB, filled once
    for (uint32_t m = 0; m < (uint32_t)kRankLutEntries; ++m) lut.mask_entry[m] = rank_lut_mask_entry(m);
    for (int i = 0; i < kTypeLutEntries; ++i) lut.type_entry[i] = rank_lut_type_entry(i / 12, (i / 4) % 3, i % 4);
    for (int i = 0; i < 8; ++i) lut.pad[i] = 0;
    RankLut* dl = nullptr;
    rc = check_cuda(cudaMalloc(&dl, sizeof(RankLut)), "cudaMalloc(rank table)");
    if (!rc) rc = check_cuda(cudaMemcpy(dl, &lut, sizeof(RankLut), cudaMemcpyHostToDevice), "cudaMemcpy(rank table)");
    if (rc) {
        cudaFree(d);
        if (dl) cudaFree(dl);
        return rc;
    }
    g_rank_lut[dev] = dl;
    g_combo[dev] = d;
    return P2B_OK;
}

const ComboTable* device_combo_table() { return g_combo[current_device()]; }
const RankLut* device_rank_lut() { return g_rank_lut[current_device()]; }

int sm_count() {
    const int dev = current_device();
    if (dev < 0 || dev >= kMaxDevices) return 148;
    if (g_sms[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        g_sms[dev] = n;
    }
    return g_sms[dev];
}

}  // namespace p2b
