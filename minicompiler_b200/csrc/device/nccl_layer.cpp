// Device layer, part 3: the collectives of the multi-GPU path.
//
// One process per GPU; weights are replicated with one broadcast at load time and
// an all-gather assembles an output only where the caller asks for it. NCCL is
// loaded at run time (dlopen of libnccl.so.2, or of the path in MCD_NCCL_LIBRARY),
// so the library carries no link-time dependency on it and a process that already
// uses NCCL shares its copy. Communicators are created non-blocking: every call is
// followed by a bounded host-side poll of the communicator's state, and a call that
// does not finish in time, or reports an asynchronous error, aborts the
// communicator (ncclCommAbort) and returns an error instead of hanging the rank.

#include "minicompiler_b200_device.h"

#include "device/driver_api.hpp"

#include <cuda_runtime_api.h>
#include <dlfcn.h>

#include <chrono>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>

#if __has_include(<nccl.h>)
#include <nccl.h>
#define MCD_HAVE_NCCL_HEADER 1
#else
#define MCD_HAVE_NCCL_HEADER 0
#endif

using namespace mcd;

#if MCD_HAVE_NCCL_HEADER

namespace {

struct NcclApi {
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRankConfig)(ncclComm_t*, int, ncclUniqueId, int, ncclConfig_t*) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*Broadcast)(const void*, void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    bool fake = false;
};

// ---- a stand-in for host-only tests: no GPU, no network, failures on demand
struct FakeState {
    std::string failing_call;
    int error_code = 0;
    bool stay_in_progress = false;
    int aborts = 0;
} g_fake;

ncclResult_t fake_result(const char* call) {
    return g_fake.failing_call == call ? static_cast<ncclResult_t>(g_fake.error_code) : ncclSuccess;
}
ncclResult_t fake_get_unique_id(ncclUniqueId* id) {
    std::memset(id, 0x5a, sizeof *id);
    return fake_result("ncclGetUniqueId");
}
ncclResult_t fake_init(ncclComm_t* comm, int, ncclUniqueId, int, ncclConfig_t*) {
    *comm = reinterpret_cast<ncclComm_t>(&g_fake);
    const ncclResult_t rc = fake_result("ncclCommInitRankConfig");
    return rc != ncclSuccess ? rc : (g_fake.stay_in_progress ? ncclInProgress : ncclSuccess);
}
ncclResult_t fake_async(ncclComm_t, ncclResult_t* state) {
    const ncclResult_t rc = fake_result("ncclCommGetAsyncError");
    *state = rc != ncclSuccess ? rc : (g_fake.stay_in_progress ? ncclInProgress : ncclSuccess);
    return ncclSuccess;
}
ncclResult_t fake_abort(ncclComm_t) {
    ++g_fake.aborts;
    return ncclSuccess;
}
ncclResult_t fake_destroy(ncclComm_t) { return fake_result("ncclCommDestroy"); }
ncclResult_t fake_broadcast(const void*, void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) {
    return fake_result("ncclBroadcast");
}
ncclResult_t fake_all_gather(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) {
    return fake_result("ncclAllGather");
}
const char* fake_error_string(ncclResult_t rc) {
    switch (rc) {
        case ncclSuccess: return "no error";
        case ncclUnhandledCudaError: return "unhandled cuda error";
        case ncclSystemError: return "unhandled system error";
        case ncclInternalError: return "internal error";
        case ncclInvalidArgument: return "invalid argument";
        case ncclInvalidUsage: return "invalid usage";
        case ncclRemoteError: return "remote process exited or there was a network error";
        case ncclInProgress: return "NCCL operation in progress";
        default: return "unknown result code";
    }
}

std::mutex g_api_mutex;
NcclApi g_api;
bool g_api_tried = false;
std::string g_api_error;

const NcclApi* nccl_api() {
    std::lock_guard<std::mutex> lock(g_api_mutex);
    if (g_api.fake || g_api.GetUniqueId != nullptr) return &g_api;
    if (g_api_tried) return nullptr;
    g_api_tried = true;
    const char* override_path = std::getenv("MCD_NCCL_LIBRARY");
    void* handle = nullptr;
    for (const char* name : {override_path, "libnccl.so.2", "libnccl.so"}) {
        if (name == nullptr || *name == '\0') continue;
        handle = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
        if (handle != nullptr) break;
        g_api_error = dlerror();
    }
    if (handle == nullptr) return nullptr;
    NcclApi api;
    bool ok = true;
    auto resolve = [&](const char* symbol, auto& slot) {
        void* fn = dlsym(handle, symbol);
        if (fn == nullptr) {
            ok = false;
            g_api_error = std::string("libnccl lacks ") + symbol;
            return;
        }
        slot = reinterpret_cast<std::remove_reference_t<decltype(slot)>>(fn);
    };
    resolve("ncclGetUniqueId", api.GetUniqueId);
    resolve("ncclCommInitRankConfig", api.CommInitRankConfig);
    resolve("ncclCommGetAsyncError", api.CommGetAsyncError);
    resolve("ncclCommAbort", api.CommAbort);
    resolve("ncclCommDestroy", api.CommDestroy);
    resolve("ncclBroadcast", api.Broadcast);
    resolve("ncclAllGather", api.AllGather);
    resolve("ncclGetErrorString", api.GetErrorString);
    if (!ok) return nullptr;
    g_api = api;
    return &g_api;
}

struct Comm {
    ncclComm_t comm = nullptr;
    int world = 1;
    int rank = 0;
    int device = 0;
    double timeout_s = 30.0;
    bool aborted = false;
    bool fake = false;
};

int nccl_fail(const NcclApi* api, const char* call, ncclResult_t rc) {
    return fail(std::string(call) + ": " + (api->GetErrorString != nullptr ? api->GetErrorString(rc) : "error") + " (NCCL result " +
                std::to_string(static_cast<int>(rc)) + ")");
}

int abort_comm(const NcclApi* api, Comm* c, const std::string& why) {
    if (!c->aborted && c->comm != nullptr) api->CommAbort(c->comm);
    c->aborted = true;
    return fail(why + "; the communicator was aborted");
}

// After a call on a non-blocking communicator: poll until it leaves the in-progress state, bounded.
int settle(const NcclApi* api, Comm* c, const char* call, ncclResult_t rc) {
    if (rc != ncclSuccess && rc != ncclInProgress) {
        const int code = nccl_fail(api, call, rc);
        const std::string text = mcd_last_error();
        if (c->comm != nullptr) return abort_comm(api, c, text);
        return code;
    }
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::duration<double>(c->timeout_s);
    for (;;) {
        ncclResult_t state = ncclSuccess;
        const ncclResult_t query = api->CommGetAsyncError(c->comm, &state);
        if (query != ncclSuccess) return abort_comm(api, c, std::string(call) + ": ncclCommGetAsyncError failed");
        if (state == ncclSuccess) return 0;
        if (state != ncclInProgress) {
            nccl_fail(api, call, state);
            return abort_comm(api, c, mcd_last_error());
        }
        if (std::chrono::steady_clock::now() > deadline) {
            char text[160];
            std::snprintf(text, sizeof text, "%s did not complete within %.1f s (rank %d of %d)", call, c->timeout_s, c->rank, c->world);
            return abort_comm(api, c, text);
        }
        std::this_thread::sleep_for(std::chrono::microseconds(c->fake ? 200 : 50));
    }
}

Comm* usable(void* comm, const char* call) {
    Comm* c = static_cast<Comm*>(comm);
    if (c == nullptr) {
        fail(std::string(call) + ": null communicator");
        return nullptr;
    }
    if (c->aborted) {
        fail(std::string(call) + ": the communicator was aborted by an earlier failure");
        return nullptr;
    }
    return c;
}

}  // namespace

extern "C" {

int mcd_nccl_available(void) { return nccl_api() != nullptr ? 1 : 0; }

int mcd_nccl_install_fake(const char* failing_call, int error_code, int stay_in_progress) {
    std::lock_guard<std::mutex> lock(g_api_mutex);
    g_fake.failing_call = failing_call != nullptr ? failing_call : "";
    g_fake.error_code = error_code;
    g_fake.stay_in_progress = stay_in_progress != 0;
    g_fake.aborts = 0;
    NcclApi api;
    api.GetUniqueId = fake_get_unique_id;
    api.CommInitRankConfig = fake_init;
    api.CommGetAsyncError = fake_async;
    api.CommAbort = fake_abort;
    api.CommDestroy = fake_destroy;
    api.Broadcast = fake_broadcast;
    api.AllGather = fake_all_gather;
    api.GetErrorString = fake_error_string;
    api.fake = true;
    g_api = api;
    return 0;
}

int mcd_nccl_remove_fake(void) {
    std::lock_guard<std::mutex> lock(g_api_mutex);
    g_api = NcclApi{};
    g_api_tried = false;
    return 0;
}

int mcd_nccl_fake_aborts(void) { return g_fake.aborts; }

int mcd_nccl_unique_id(char* id) {
    const NcclApi* api = nccl_api();
    if (api == nullptr) return fail("NCCL is unavailable: " + g_api_error);
    static_assert(sizeof(ncclUniqueId) == MCD_NCCL_ID_BYTES, "size of an NCCL unique id");
    ncclUniqueId uid;
    const ncclResult_t rc = api->GetUniqueId(&uid);
    if (rc != ncclSuccess) return nccl_fail(api, "ncclGetUniqueId", rc);
    std::memcpy(id, &uid, sizeof uid);
    return 0;
}

int mcd_nccl_init(void** comm, int world_size, int rank, const char* id, int device, double timeout_s) {
    *comm = nullptr;
    const NcclApi* api = nccl_api();
    if (api == nullptr) return fail("NCCL is unavailable: " + g_api_error);
    if (world_size < 1 || rank < 0 || rank >= world_size) return fail("mcd_nccl_init: rank outside the world");
    if (!api->fake) {
        if (int rc = check_rt(cudaSetDevice(device), "cudaSetDevice")) return rc;
    }
    auto* c = new Comm();
    c->world = world_size;
    c->rank = rank;
    c->device = device;
    c->timeout_s = timeout_s > 0.0 ? timeout_s : 30.0;
    c->fake = api->fake;
    ncclUniqueId uid;
    std::memcpy(&uid, id, sizeof uid);
    ncclConfig_t config = NCCL_CONFIG_INITIALIZER;
    config.blocking = 0;
    const ncclResult_t rc = api->CommInitRankConfig(&c->comm, world_size, uid, rank, &config);
    if (int failed = settle(api, c, "ncclCommInitRankConfig", rc)) {
        delete c;
        return failed;
    }
    *comm = c;
    return 0;
}

int mcd_nccl_broadcast(void* comm, void* buffer, size_t bytes, int root, void* stream) {
    const NcclApi* api = nccl_api();
    Comm* c = usable(comm, "mcd_nccl_broadcast");
    if (api == nullptr || c == nullptr) return 1;
    if (root < 0 || root >= c->world) return fail("mcd_nccl_broadcast: root outside the world");
    if (bytes == 0) return 0;
    const ncclResult_t rc = api->Broadcast(buffer, buffer, bytes, ncclInt8, root, c->comm, static_cast<cudaStream_t>(stream));
    return settle(api, c, "ncclBroadcast", rc);
}

int mcd_nccl_all_gather(void* comm, const void* send, void* recv, size_t bytes_per_rank, void* stream) {
    const NcclApi* api = nccl_api();
    Comm* c = usable(comm, "mcd_nccl_all_gather");
    if (api == nullptr || c == nullptr) return 1;
    if (bytes_per_rank == 0) return 0;
    const ncclResult_t rc = api->AllGather(send, recv, bytes_per_rank, ncclInt8, c->comm, static_cast<cudaStream_t>(stream));
    return settle(api, c, "ncclAllGather", rc);
}

int mcd_nccl_wait(void* comm, void* stream) {
    const NcclApi* api = nccl_api();
    Comm* c = usable(comm, "mcd_nccl_wait");
    if (api == nullptr || c == nullptr) return 1;
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::duration<double>(c->timeout_s);
    for (;;) {
        ncclResult_t state = ncclSuccess;
        if (api->CommGetAsyncError(c->comm, &state) != ncclSuccess) return abort_comm(api, c, "mcd_nccl_wait: ncclCommGetAsyncError failed");
        if (state != ncclSuccess && state != ncclInProgress) {
            nccl_fail(api, "a collective", state);
            return abort_comm(api, c, mcd_last_error());
        }
        bool done = state == ncclSuccess;
        if (done && !c->fake) {
            const cudaError_t q = cudaStreamQuery(static_cast<cudaStream_t>(stream));
            if (q == cudaErrorNotReady) {
                done = false;
            } else if (q != cudaSuccess) {
                return check_rt(q, "cudaStreamQuery");
            }
        }
        if (done) return 0;
        if (std::chrono::steady_clock::now() > deadline) {
            char text[160];
            std::snprintf(text, sizeof text, "the collectives on this stream did not complete within %.1f s (rank %d of %d)", c->timeout_s,
                          c->rank, c->world);
            return abort_comm(api, c, text);
        }
        std::this_thread::sleep_for(std::chrono::microseconds(c->fake ? 200 : 50));
    }
}

int mcd_nccl_abort(void* comm) {
    const NcclApi* api = nccl_api();
    Comm* c = static_cast<Comm*>(comm);
    if (api == nullptr || c == nullptr) return 0;
    if (!c->aborted && c->comm != nullptr) api->CommAbort(c->comm);
    c->aborted = true;
    return 0;
}

int mcd_nccl_destroy(void* comm) {
    const NcclApi* api = nccl_api();
    Comm* c = static_cast<Comm*>(comm);
    if (c == nullptr) return 0;
    int rc = 0;
    if (api != nullptr && !c->aborted && c->comm != nullptr) {
        const ncclResult_t r = api->CommDestroy(c->comm);
        if (r != ncclSuccess && r != ncclInProgress) rc = nccl_fail(api, "ncclCommDestroy", r);
    }
    delete c;
    return rc;
}

}  // extern "C"

#else  // no NCCL header at build time: the entry points exist and say so

extern "C" {
int mcd_nccl_available(void) { return 0; }
int mcd_nccl_install_fake(const char*, int, int) { return fail("built without nccl.h"); }
int mcd_nccl_remove_fake(void) { return 0; }
int mcd_nccl_fake_aborts(void) { return 0; }
int mcd_nccl_unique_id(char*) { return fail("NCCL is unavailable: built without nccl.h"); }
int mcd_nccl_init(void** comm, int, int, const char*, int, double) {
    *comm = nullptr;
    return fail("NCCL is unavailable: built without nccl.h");
}
int mcd_nccl_broadcast(void*, void*, size_t, int, void*) { return fail("NCCL is unavailable: built without nccl.h"); }
int mcd_nccl_all_gather(void*, const void*, void*, size_t, void*) { return fail("NCCL is unavailable: built without nccl.h"); }
int mcd_nccl_wait(void*, void*) { return fail("NCCL is unavailable: built without nccl.h"); }
int mcd_nccl_abort(void*) { return 0; }
int mcd_nccl_destroy(void*) { return 0; }
}

#endif
