// Opens the kernel libraries and resolves their entry points (kernels.h).
#include "ops/kernels.h"

#include <dlfcn.h>
#include <stdlib.h>
#include <sys/stat.h>

#include <map>
#include <mutex>

#include "friday/base.h"

namespace friday {
namespace kernels {

namespace {
std::mutex g_mutex;
builder_fn g_builder = nullptr;
std::map<std::string, void*> g_handles;
std::map<std::string, std::string> g_paths;

bool exists(const std::string& p) {
    struct stat st;
    return stat(p.c_str(), &st) == 0;
}

void* open_family(const std::string& family) {
    auto it = g_handles.find(family);
    if (it != g_handles.end()) return it->second;
    // The builder decides whether the library on disk was made from the present sources.
    if (g_builder && g_builder(family.c_str()) != 0)
        throw KernelError("the kernel library '" + family + "' could not be built (see the builder's message above)");
    const std::string path = library_dir() + "/libfriday_" + family + ".so";
    if (!exists(path))
        throw KernelError("kernel library " + path + " is missing and nothing is set up to build it: run "
                          "`python -m friday_inference_engine_b200.ops.build` (needs nvcc), or set FRIDAY_BUILD_DIR "
                          "to the folder that holds the built libraries; there is no other path");
    void* h = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (!h) throw KernelError("cannot load " + path + ": " + dlerror());
    g_handles[family] = h;
    g_paths[family] = path;
    return h;
}

template <class F> void resolve(void* h, const std::string& family, const char* name, F& out) {
    void* s = dlsym(h, name);
    if (!s) throw KernelError("kernel library '" + family + "' has no entry point " + name);
    out = (F)s;
}
}  // namespace

void set_builder(builder_fn f) {
    std::lock_guard<std::mutex> lock(g_mutex);
    g_builder = f;
}

std::string library_dir() {
    const char* env = getenv("FRIDAY_BUILD_DIR");
    if (env && env[0]) return env;
    Dl_info info;
    if (dladdr((void*)&library_dir, &info) && info.dli_fname) {
        std::string p = info.dli_fname;
        size_t slash = p.rfind('/');
        return slash == std::string::npos ? "." : p.substr(0, slash);
    }
    return ".";
}

std::string loaded_libraries() {
    std::lock_guard<std::mutex> lock(g_mutex);
    std::string out;
    for (const auto& kv : g_paths) out += kv.second + "\n";
    return out;
}

#define FAMILY(Type, fn, family, ...)                          \
    const Type& fn() {                                         \
        static Type t;                                         \
        static bool ready = false;                             \
        std::lock_guard<std::mutex> lock(g_mutex);             \
        if (!ready) {                                          \
            void* h = open_family(family);                     \
            const std::string fam = family;                    \
            resolve(h, fam, family "_last_error", t.last_error); \
            __VA_ARGS__                                        \
            ready = true;                                      \
        }                                                      \
        return t;                                              \
    }

FAMILY(Rowwise, rowwise, "rowwise",
       resolve(h, fam, "rowwise_embedding", t.embedding); resolve(h, fam, "rowwise_gather_rows", t.gather_rows);
       resolve(h, fam, "rowwise_rmsnorm", t.rmsnorm); resolve(h, fam, "rowwise_swiglu", t.swiglu);
       resolve(h, fam, "rowwise_rope_kv_write", t.rope_kv_write); resolve(h, fam, "rowwise_advance", t.advance);
       resolve(h, fam, "rowwise_scale_rows", t.scale_rows); resolve(h, fam, "rowwise_finish_logits", t.finish_logits);
       resolve(h, fam, "rowwise_random_normal", t.random_normal);)
FAMILY(GemmSimt, gemm_simt, "gemm_simt", resolve(h, fam, "gemm_simt", t.gemm);)
FAMILY(GemmTc, gemm_tc, "gemm_tc", resolve(h, fam, "gemm_tc_fused", t.fused); resolve(h, fam, "gemm_tc_plan", t.plan);)
FAMILY(AttentionSimt, attention_simt, "attention_simt", resolve(h, fam, "attention_simt", t.run);)
FAMILY(AttentionMma, attention_mma, "attention_mma", resolve(h, fam, "attention_mma", t.run);
       resolve(h, fam, "attention_mma_clusters_at_once", t.clusters_at_once);)
FAMILY(AttentionTc, attention_tc, "attention_tc", resolve(h, fam, "attention_tc", t.run);)
FAMILY(Sampling, sampling, "sampling", resolve(h, fam, "sampling_sample", t.sample);)

}  // namespace kernels
}  // namespace friday
