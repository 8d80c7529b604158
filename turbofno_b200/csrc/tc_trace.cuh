// Per-role cycle counters of spectral_tc_kernel, host side.  Compiled only with -DTFNO_TC_TRACE
// (a diagnostic build: it allocates a counter buffer, synchronises the device after every fused
// launch and prints one line per warp role to stderr).  Release builds do not include this file.
// Included by launch.cuh inside namespace tfno, after DeviceInfo.
#pragma once
#ifdef TFNO_TC_TRACE

constexpr int kTraceWarps = 24, kTraceSlots = 12;

// counter buffer of the device, sized from its SM count; cleared when `clear` is set
inline long long* tc_trace_buffer(const DeviceInfo& dev, bool clear) {
    static long long* buf[64] = {};
    const size_t bytes = sizeof(long long) * (size_t)dev.sms * kTraceWarps * kTraceSlots;
    if (dev.device < 0 || dev.device >= 64) return nullptr;
    if (!buf[dev.device] && cudaMalloc(&buf[dev.device], bytes) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    if (clear) cudaMemset(buf[dev.device], 0, bytes);
    return buf[dev.device];
}

// mean over the CTAs of a launch, one line per warp
inline void tc_trace_report(const DeviceInfo& dev, int grid) {
    long long* buf = tc_trace_buffer(dev, false);
    if (!buf || grid <= 0) return;
    cudaDeviceSynchronize();
    std::vector<long long> host((size_t)dev.sms * kTraceWarps * kTraceSlots);
    cudaMemcpy(host.data(), buf, host.size() * sizeof(long long), cudaMemcpyDeviceToHost);
    const char* role[kTraceWarps] = {"F0", "I1", "F2", "I3", "F4", "I5", "F6", "I7", "F8", "I9", "F10", "I11", "F12", "I13", "F14", "I15",
                                     "X16", "X17", "X18", "X19", "PROD", "MMA", "-", "-"};
    for (int w = 0; w < kTraceWarps; ++w) {
        double t[kTraceSlots] = {};
        for (int b = 0; b < grid; ++b)
            for (int k = 0; k < kTraceSlots; ++k) t[k] += (double)host[((size_t)b * kTraceWarps + w) * kTraceSlots + k] / grid;
        std::fprintf(stderr, "trace %-4s total=%8.0f w0=%7.0f w1=%7.0f w2=%7.0f w3=%7.0f load=%7.0f mma=%7.0f fft=%7.0f in=%7.0f mid=%7.0f out=%7.0f loop=%7.0f\n",
                     role[w], t[0], t[1], t[2], t[3], t[4], t[5], t[6], t[7], t[8], t[9], t[10], t[11]);
    }
}

#endif
