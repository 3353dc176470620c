// Kernel-launch counter built on CUPTI driver-API callbacks: begin_launch_trace() subscribes, every
// cuLaunch* / cuGraphLaunch* entered until end_launch_trace() is counted and the first kernel symbol is kept.
// libcupti is opened with dlopen at first use, so this library loads on machines without CUPTI and
// reports CUPTI_ERROR_NOT_INITIALIZED (15) from begin_launch_trace instead.
#include <cupti.h>
#include <dlfcn.h>

#include <atomic>
#include <cstring>
#include <mutex>
#include <string>

namespace {

struct Api {
    CUptiResult (*subscribe)(CUpti_SubscriberHandle*, CUpti_CallbackFunc, void*) = nullptr;
    CUptiResult (*unsubscribe)(CUpti_SubscriberHandle) = nullptr;
    CUptiResult (*enable_domain)(uint32_t, CUpti_SubscriberHandle, CUpti_CallbackDomain) = nullptr;
    CUptiResult (*result_string)(CUptiResult, const char**) = nullptr;
    bool ok = false;
};

Api& api() {
    static Api a;
    static std::once_flag once;
    std::call_once(once, [] {
        const char* names[] = {"libcupti.so", "libcupti.so.12", "/usr/local/cuda/lib64/libcupti.so",
                               "/usr/local/cuda/extras/CUPTI/lib64/libcupti.so"};
        void* lib = nullptr;
        for (const char* n : names)
            if ((lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL))) break;
        if (!lib) return;
        a.subscribe = reinterpret_cast<decltype(a.subscribe)>(dlsym(lib, "cuptiSubscribe"));
        a.unsubscribe = reinterpret_cast<decltype(a.unsubscribe)>(dlsym(lib, "cuptiUnsubscribe"));
        a.enable_domain = reinterpret_cast<decltype(a.enable_domain)>(dlsym(lib, "cuptiEnableDomain"));
        a.result_string = reinterpret_cast<decltype(a.result_string)>(dlsym(lib, "cuptiGetResultString"));
        a.ok = a.subscribe && a.unsubscribe && a.enable_domain;
    });
    return a;
}

struct Trace {
    CUpti_SubscriberHandle subscriber{};
    std::atomic<int> launches{0};
    std::mutex lock;
    std::string first_symbol;
};

bool is_launch(CUpti_CallbackId id) {
    switch (id) {
        case CUPTI_DRIVER_TRACE_CBID_cuLaunch:
        case CUPTI_DRIVER_TRACE_CBID_cuLaunchGrid:
        case CUPTI_DRIVER_TRACE_CBID_cuLaunchGridAsync:
        case CUPTI_DRIVER_TRACE_CBID_cuLaunchKernel:
        case CUPTI_DRIVER_TRACE_CBID_cuLaunchKernel_ptsz:
        case CUPTI_DRIVER_TRACE_CBID_cuLaunchKernelEx:
        case CUPTI_DRIVER_TRACE_CBID_cuLaunchKernelEx_ptsz:
        case CUPTI_DRIVER_TRACE_CBID_cuLaunchCooperativeKernel:
        case CUPTI_DRIVER_TRACE_CBID_cuLaunchCooperativeKernel_ptsz:
        case CUPTI_DRIVER_TRACE_CBID_cuLaunchCooperativeKernelMultiDevice:
        case CUPTI_DRIVER_TRACE_CBID_cuGraphLaunch:
        case CUPTI_DRIVER_TRACE_CBID_cuGraphLaunch_ptsz:
            return true;
        default:
            return false;
    }
}

void CUPTIAPI on_callback(void* user, CUpti_CallbackDomain domain, CUpti_CallbackId id, const void* data) {
    if (domain != CUPTI_CB_DOMAIN_DRIVER_API || !is_launch(id)) return;
    const auto* info = static_cast<const CUpti_CallbackData*>(data);
    if (info->callbackSite != CUPTI_API_ENTER) return;
    auto* trace = static_cast<Trace*>(user);
    if (trace->launches.fetch_add(1) == 0 && info->symbolName) {
        std::lock_guard<std::mutex> guard(trace->lock);
        trace->first_symbol = info->symbolName;
    }
}

}  // namespace

extern "C" int begin_launch_trace(void** handle) {
    if (!handle) return CUPTI_ERROR_INVALID_PARAMETER;
    *handle = nullptr;
    Api& a = api();
    if (!a.ok) return CUPTI_ERROR_NOT_INITIALIZED;
    auto* trace = new Trace();
    CUptiResult r = a.subscribe(&trace->subscriber, on_callback, trace);
    if (r == CUPTI_SUCCESS) r = a.enable_domain(1, trace->subscriber, CUPTI_CB_DOMAIN_DRIVER_API);
    if (r != CUPTI_SUCCESS) {
        if (trace->subscriber) a.unsubscribe(trace->subscriber);
        delete trace;
        return r;
    }
    *handle = trace;
    return CUPTI_SUCCESS;
}

extern "C" int end_launch_trace(void* handle, int* count, char* symbol, int symbol_bytes) {
    if (!handle || !count) return CUPTI_ERROR_INVALID_PARAMETER;
    auto* trace = static_cast<Trace*>(handle);
    CUptiResult r = api().unsubscribe(trace->subscriber);
    *count = trace->launches.load();
    if (symbol && symbol_bytes > 0) {
        std::strncpy(symbol, trace->first_symbol.c_str(), static_cast<size_t>(symbol_bytes) - 1);
        symbol[symbol_bytes - 1] = '\0';
    }
    delete trace;
    return r;
}

extern "C" const char* launch_trace_error(int code) {
    const char* text = "unknown CUPTI error";
    Api& a = api();
    if (a.result_string) a.result_string(static_cast<CUptiResult>(code), &text);
    return text;
}
