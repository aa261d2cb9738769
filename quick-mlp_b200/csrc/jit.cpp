// Per-spec kernel instantiation: hash the generated source together with the kernel template headers, look the
// shared object up in the cache directory, otherwise build it with nvcc for sm_100a, then dlopen it.
// This replaces the reference's run-time NVRTC path (ckl::KernelLoader::getKernel, used at
// src_cpp/src/fused_network.cpp:465-470 and src_cpp/src/iencoding.cpp:59-63) and its on-disk kernel cache.
#include "host.hpp"

#include <atomic>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <dirent.h>
#include <dlfcn.h>
#include <fstream>
#include <sstream>
#include <sys/stat.h>
#include <unistd.h>

#include <cuda_runtime.h>

#include "generic_kernels.h"

namespace qmlp {

Library& Library::instance()
{
    static Library lib;
    return lib;
}

void logMessage(int level, const std::string& msg)
{
    Library& lib = Library::instance();
    if (level < lib.logLevel) return;
    static const char* names[] = {"debug", "info", "warning", "error"};
    std::fprintf(stderr, "[qmlp] [%s] %s\n", names[level < 0 ? 0 : level > 3 ? 3 : level], msg.c_str());
}

static std::string dirOfThisLibrary()
{
    Dl_info info;
    if (dladdr(reinterpret_cast<void*>(&dirOfThisLibrary), &info) && info.dli_fname) {
        std::string p = info.dli_fname;
        size_t s = p.find_last_of('/');
        return s == std::string::npos ? std::string(".") : p.substr(0, s);
    }
    return ".";
}

static bool isDir(const std::string& p)
{
    struct stat st;
    return ::stat(p.c_str(), &st) == 0 && S_ISDIR(st.st_mode);
}

static void makeDirs(const std::string& p)
{
    std::string cur;
    for (size_t i = 0; i < p.size(); ++i) {
        cur += p[i];
        if (p[i] == '/' || i + 1 == p.size()) ::mkdir(cur.c_str(), 0755);
    }
}

std::string Library::resolveCacheDir()
{
    if (!cacheDir.empty()) return cacheDir;
    if (const char* e = std::getenv("QMLP_KERNEL_CACHE")) cacheDir = e;
    else cacheDir = dirOfThisLibrary() + "/specs";
    return cacheDir;
}

std::string Library::resolveIncludeDir()
{
    if (!includeDir.empty()) return includeDir;
    if (const char* e = std::getenv("QMLP_KERNEL_INCLUDE")) { includeDir = e; return includeDir; }
    const std::string base = dirOfThisLibrary();
    for (const char* rel : {"/../csrc/kernels", "/kernels", "/csrc/kernels"}) {
        if (isDir(base + rel)) { includeDir = base + rel; return includeDir; }
    }
    includeDir = base + "/../csrc/kernels";
    return includeDir;
}

int Library::smCount()
{
    static std::atomic<int> cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) throw cuda_error("cudaGetDevice failed: no CUDA device available");
    if (dev < 0 || dev >= 64) throw cuda_error("device index out of range (at most 64 devices per process)");
    int n = cached[dev].load(std::memory_order_relaxed);
    if (n == 0) {
        cudaError_t e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) throw cuda_error(std::string("cudaDeviceGetAttribute: ") + cudaGetErrorString(e));
        cached[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

int* Library::statusWord()
{
    static std::atomic<int*> words[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) throw cuda_error("cudaGetDevice failed: no CUDA device available");
    if (dev < 0 || dev >= 64) throw cuda_error("device index out of range (at most 64 devices per process)");
    int* w = words[dev].load(std::memory_order_acquire);
    if (w == nullptr) {
        // the word is a __device__ variable of this library (zero at module load): nothing is allocated
        cudaError_t e = kernel::statusWordAddress(&w);
        if (e != cudaSuccess) throw cuda_error(std::string("status word lookup failed: ") + cudaGetErrorString(e));
        words[dev].store(w, std::memory_order_release);
    }
    return w;
}

static uint64_t fnv1a(const std::string& s, uint64_t h = 1469598103934665603ULL)
{
    for (unsigned char c : s) { h ^= c; h *= 1099511628211ULL; }
    return h;
}

static std::string readFile(const std::string& p)
{
    std::ifstream in(p, std::ios::binary);
    std::stringstream ss;
    ss << in.rdbuf();
    return ss.str();
}

// digest of every kernel template header, so a header change invalidates cached instantiations
static uint64_t headersDigest(const std::string& dir)
{
    static std::map<std::string, uint64_t> cache;
    auto it = cache.find(dir);
    if (it != cache.end()) return it->second;
    std::vector<std::string> names;
    if (DIR* d = ::opendir(dir.c_str())) {
        while (dirent* e = ::readdir(d)) {
            std::string n = e->d_name;
            if (n.size() > 2 && (n.rfind(".cuh") == n.size() - 4 || n.rfind(".h") == n.size() - 2)) names.push_back(n);
        }
        ::closedir(d);
    }
    if (names.empty()) throw compile_error("kernel template headers not found in '" + dir + "' (set QMLP_KERNEL_INCLUDE)");
    std::sort(names.begin(), names.end());
    uint64_t h = 1469598103934665603ULL;
    for (const auto& n : names) h = fnv1a(readFile(dir + "/" + n), fnv1a(n, h));
    cache[dir] = h;
    return h;
}

static std::map<std::string, std::shared_ptr<KernelModule>>& registry()
{
    static std::map<std::string, std::shared_ptr<KernelModule>> r;
    return r;
}

static std::shared_ptr<KernelModule> loadModule(const std::string& name, const std::string& path)
{
    void* h = ::dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (!h) throw compile_error(std::string("dlopen failed for '") + path + "': " + ::dlerror());
    auto abi = reinterpret_cast<qmlp_spec_abi_fn>(::dlsym(h, "qmlp_spec_abi"));
    auto launch = reinterpret_cast<qmlp_spec_launch_fn>(::dlsym(h, "qmlp_spec_launch"));
    if (!abi || !launch || abi() != QMLP_SPEC_ABI_VERSION) {
        ::dlclose(h);
        throw compile_error("instantiation '" + path + "' has the wrong ABI version; delete it to rebuild");
    }
    auto m = std::make_shared<KernelModule>();
    m->name = name;
    m->handle = h;
    m->launch = launch;
    return m;
}

std::shared_ptr<KernelModule> getKernelModule(const std::string& kind, const std::string& source)
{
    Library& lib = Library::instance();
    std::lock_guard<std::mutex> lock(lib.mutex);
    const std::string inc = lib.resolveIncludeDir();
    const std::string cache = lib.resolveCacheDir();
    uint64_t h = fnv1a(source, headersDigest(inc));
    h = fnv1a(lib.debugMode ? "debug" : "release", h);
    if (lib.boundsCheck) h = fnv1a("bounds-check", h);
    h = fnv1a(std::to_string(QMLP_SPEC_ABI_VERSION), h);
    char hex[32];
    std::snprintf(hex, sizeof hex, "%016llx", static_cast<unsigned long long>(h));
    const std::string name = "qmlp_" + kind + "_" + hex;

    auto& reg = registry();
    auto it = reg.find(name);
    if (it != reg.end()) return it->second;

    const std::string so = cache + "/" + name + ".so";
    struct stat st;
    if (::stat(so.c_str(), &st) != 0) {
        // build it
        makeDirs(cache);
        // Several processes may meet the same missing instantiation at once (one rank per GPU on a cold cache): each
        // builds from its own source, log and output file, and only the finished shared object is renamed into place.
        const std::string unique = std::to_string(::getpid());
        const std::string cu = cache + "/" + name + "." + unique + ".cu";
        const std::string tmp = so + ".tmp" + unique;
        const std::string log = cache + "/" + name + "." + unique + ".log";
        {
            std::ofstream out(cu);
            out << source;
            if (!out) throw compile_error("cannot write '" + cu + "'");
        }
        std::string nvcc = lib.nvcc;
        if (nvcc.empty()) {
            if (const char* e = std::getenv("QMLP_NVCC")) nvcc = e;
            else if (::access("/usr/local/cuda/bin/nvcc", X_OK) == 0) nvcc = "/usr/local/cuda/bin/nvcc";
            else nvcc = "nvcc";
        }
        std::ostringstream cmd;
        cmd << nvcc << " -std=c++17 -gencode arch=compute_100a,code=sm_100a -lineinfo "
            << (lib.debugMode ? "-O0 -G " : "-O3 ") << (lib.boundsCheck ? "-DQMLP_BOUNDS_CHECK " : "") << "-shared -Xcompiler -fPIC -I'" << inc << "' -o '" << tmp << "' '" << cu
            << "' > '" << log << "' 2>&1";
        logMessage(1, "instantiating kernels for a new spec: " + name + " (nvcc, this takes a few seconds)");
        const int rc = std::system(cmd.str().c_str());
        if (rc != 0) {
            std::string msg = readFile(log);
            if (msg.size() > 4000) msg = msg.substr(0, 4000) + "...";
            ::unlink(tmp.c_str());
            throw compile_error("nvcc failed for '" + cu + "' (command: " + cmd.str() + "):\n" + msg);
        }
        if (::rename(tmp.c_str(), so.c_str()) != 0) {
            ::unlink(tmp.c_str());
            throw compile_error("cannot move the built instantiation to '" + so + "'");
        }
        // keep one copy of the generated source and of the compiler log beside the shared object
        ::rename(cu.c_str(), (cache + "/" + name + ".cu").c_str());
        ::rename(log.c_str(), (cache + "/" + name + ".log").c_str());
    }
    auto m = loadModule(name, so);
    reg[name] = m;
    return m;
}

} // namespace qmlp
