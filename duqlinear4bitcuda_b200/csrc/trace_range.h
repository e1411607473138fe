// NVTX ranges around the library's entry points (host side only): a timeline tool that injects itself
// through NVTX_INJECTION64_PATH sees one range per call, named after the entry point, in the domain "duq4".
// Without a tool attached the header-only NVTX v3 stubs reduce each push/pop to a null-pointer test.
#pragma once
#include <nvtx3/nvToolsExt.h>

namespace duq4 {

inline nvtxDomainHandle_t trace_domain() {
    static nvtxDomainHandle_t d = nvtxDomainCreateA("duq4");
    return d;
}

struct TraceRange {
    explicit TraceRange(const char *name) {
        nvtxEventAttributes_t a = {};
        a.version = NVTX_VERSION;
        a.size = NVTX_EVENT_ATTRIB_STRUCT_SIZE;
        a.messageType = NVTX_MESSAGE_TYPE_ASCII;
        a.message.ascii = name;
        nvtxDomainRangePushEx(trace_domain(), &a);
    }
    ~TraceRange() { nvtxDomainRangePop(trace_domain()); }
    TraceRange(const TraceRange &) = delete;
    TraceRange &operator=(const TraceRange &) = delete;
};

}  // namespace duq4

#define DUQ4_TRACE() ::duq4::TraceRange duq4_trace_range_(__func__)
