#include "nccl_dl.h"

#include <dlfcn.h>

#include <cstdlib>
#include <mutex>
#include <string>

namespace ava {

namespace {
NcclApi g_api{};
bool g_ok = false;
std::string g_err;
std::once_flag g_once;

void load() {
    const char* names[3] = {std::getenv("AVA_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
    void* h = nullptr;
    for (const char* n : names) {
        if (!n || !*n) continue;
        h = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (h) break;
        g_err = dlerror();
    }
    if (!h) {
        if (g_err.empty()) g_err = "no NCCL library found";
        return;
    }
    auto sym = [&](const char* n) -> void* {
        void* p = dlsym(h, n);
        if (!p) g_err = std::string("NCCL symbol missing: ") + n;
        return p;
    };
    g_api.GetUniqueId = reinterpret_cast<decltype(g_api.GetUniqueId)>(sym("ncclGetUniqueId"));
    g_api.CommInitRank = reinterpret_cast<decltype(g_api.CommInitRank)>(sym("ncclCommInitRank"));
    g_api.CommDestroy = reinterpret_cast<decltype(g_api.CommDestroy)>(sym("ncclCommDestroy"));
    g_api.Broadcast = reinterpret_cast<decltype(g_api.Broadcast)>(sym("ncclBroadcast"));
    g_api.AllGather = reinterpret_cast<decltype(g_api.AllGather)>(sym("ncclAllGather"));
    g_api.GetErrorString = reinterpret_cast<decltype(g_api.GetErrorString)>(sym("ncclGetErrorString"));
    g_api.GetVersion = reinterpret_cast<decltype(g_api.GetVersion)>(sym("ncclGetVersion"));
    g_api.CommGetAsyncError = reinterpret_cast<decltype(g_api.CommGetAsyncError)>(dlsym(h, "ncclCommGetAsyncError"));
    g_api.CommAbort = reinterpret_cast<decltype(g_api.CommAbort)>(dlsym(h, "ncclCommAbort"));
    g_ok = g_api.GetUniqueId && g_api.CommInitRank && g_api.CommDestroy && g_api.Broadcast && g_api.AllGather && g_api.GetErrorString && g_api.GetVersion;
}
}  // namespace

const NcclApi* nccl_api() {
    std::call_once(g_once, load);
    return g_ok ? &g_api : nullptr;
}
const char* nccl_dl_error() { return g_err.c_str(); }

}  // namespace ava
