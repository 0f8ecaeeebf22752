// Run-time specialisation of the broadcast evaluator.
//
// The reference compiles every broadcast expression to native code with its Julia-to-GPU
// compiler.  This library ships ahead-of-time kernels: hard-wired ones for the common trees and
// an interpreter (program.cuh) for everything else.  The interpreter is instruction bound (an
// indirect branch, a dozen register moves and a run-time element-type switch per operator and
// vector).  Here the SAME evaluator source is compiled once per distinct expression with the
// program as a compile-time constant (NVRTC, cubin for sm_100a): loops unroll, every switch
// folds, the result is straight-line code that streams at the speed of the hard-wired kernels
// and computes bit for bit what the interpreter computes.  Compiled kernels are cached by the
// expression's structure (operators, element types, layout flags; pointers, shapes and scalar
// values stay run-time arguments).  NVRTC is loaded with dlopen; when it is missing, or a
// compilation fails, the interpreter runs instead - still on the GPU.
#include "reduce_program.cuh"

#include <dlfcn.h>
#include <nvrtc.h>

#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "rtc_sources.inc"   // kRtcCommon, kRtcProgram, kRtcReduce, kRtcHeader: the sources as strings

namespace b200 {

namespace {

struct Nvrtc {
    void* handle = nullptr;
    bool tried = false;
    nvrtcResult (*CreateProgram)(nvrtcProgram*, const char*, const char*, int, const char* const*, const char* const*) = nullptr;
    nvrtcResult (*CompileProgram)(nvrtcProgram, int, const char* const*) = nullptr;
    nvrtcResult (*GetCUBINSize)(nvrtcProgram, size_t*) = nullptr;
    nvrtcResult (*GetCUBIN)(nvrtcProgram, char*) = nullptr;
    nvrtcResult (*GetProgramLogSize)(nvrtcProgram, size_t*) = nullptr;
    nvrtcResult (*GetProgramLog)(nvrtcProgram, char*) = nullptr;
    nvrtcResult (*DestroyProgram)(nvrtcProgram*) = nullptr;
};

struct Entry {
    std::vector<char> cubin;         // empty: compilation failed, do not try again
    cudaLibrary_t lib = nullptr;     // loaded on first launch
    cudaKernel_t kernel = nullptr;
    int blocks_per_sm = 0;
};

std::mutex g_mu;
Nvrtc g_nvrtc;
std::map<std::string, Entry> g_cache;
int g_enabled = -1;                  // -1: not decided yet (environment), 0 / 1
uint64_t g_compiled = 0, g_hits = 0, g_failures = 0;
std::string g_last_log;

bool load_nvrtc() {
    if (g_nvrtc.tried) return g_nvrtc.handle != nullptr;
    g_nvrtc.tried = true;
    const char* names[] = {getenv("B200_NVRTC_LIB"), "libnvrtc.so.12", "/usr/local/cuda/lib64/libnvrtc.so.12",
                           "/usr/local/cuda/lib64/libnvrtc.so", "libnvrtc.so"};
    void* h = nullptr;
    for (const char* n : names) {
        if (!n || !*n) continue;
        h = dlopen(n, RTLD_NOW | RTLD_LOCAL);
        if (h) break;
    }
    if (!h) return false;
#define B200_SYM(field, name) *(void**)(&g_nvrtc.field) = dlsym(h, name); if (!g_nvrtc.field) { dlclose(h); return false; }
    B200_SYM(CreateProgram, "nvrtcCreateProgram")
    B200_SYM(CompileProgram, "nvrtcCompileProgram")
    B200_SYM(GetCUBINSize, "nvrtcGetCUBINSize")
    B200_SYM(GetCUBIN, "nvrtcGetCUBIN")
    B200_SYM(GetProgramLogSize, "nvrtcGetProgramLogSize")
    B200_SYM(GetProgramLog, "nvrtcGetProgramLog")
    B200_SYM(DestroyProgram, "nvrtcDestroyProgram")
#undef B200_SYM
    g_nvrtc.handle = h;
    return true;
}

bool enabled() {
    if (g_enabled < 0) {
        const char* e = getenv("B200_JIT");
        g_enabled = (e && e[0] == '0') ? 0 : 1;
    }
    return g_enabled == 1;
}

// Everything the generated code depends on, and nothing else.
struct ReduceInfo { int redop, acc_dtype, full; };

std::string cache_key(const Compiled& C, int out_dtype, const ReduceInfo* red = nullptr) {
    std::string k;
    if (red) { k.push_back('R'); k.push_back((char)red->redop); k.push_back((char)red->acc_dtype); k.push_back((char)red->full); }
    else k.push_back('B');
    k.push_back(C.wide ? 'W' : 'N');
    k.push_back((char)C.P.ninstr);
    k.append(reinterpret_cast<const char*>(C.P.hcode), 2 * (size_t)C.P.ninstr);
    k.push_back((char)C.P.nleaves);
    for (int i = 0; i < C.P.nleaves; ++i) {
        k.push_back((char)C.P.leaves[i].dtype);
        k.push_back((char)(C.P.leaves[i].is_scalar ? 1 : 0));
    }
    k.push_back((char)(C.P.linear ? 1 : 0));
    k.push_back((char)(C.P.vec_ok ? 1 : 0));
    k.push_back((char)out_dtype);
    return k;
}

std::string byte_list(const unsigned char* p, int n) {
    std::string s;
    for (int i = 0; i < n; ++i) {
        if (i) s += ", ";
        s += std::to_string((int)p[i]);
    }
    return n ? s : std::string("0");
}

std::string generate_source(const Compiled& C, int out_dtype, const ReduceInfo* red = nullptr) {
    const ProgramDesc& P = C.P;
    unsigned char ld[B200_MAX_LEAVES + 1] = {0}, ls[B200_MAX_LEAVES + 1] = {0};
    for (int i = 0; i < P.nleaves; ++i) { ld[i] = (unsigned char)P.leaves[i].dtype; ls[i] = P.leaves[i].is_scalar ? 1 : 0; }
    std::string s = red ? "#include \"reduce_program.cuh\"\n" : "#include \"program.cuh\"\n";
    s += "namespace b200 {\nstruct StaticCode {\n    static constexpr bool is_static = true;\n";
    s += "    static constexpr int redop = " + std::to_string(red ? red->redop : 0) + ", acc_dtype = " +
         std::to_string(red ? red->acc_dtype : 0) + ", full = " + std::to_string(red ? red->full : 0) + ";\n";
    s += "    static constexpr int ninstr = " + std::to_string(P.ninstr) + ", nleaves = " + std::to_string(P.nleaves) +
         ", linear = " + std::to_string(P.linear ? 1 : 0) + ", vec_ok = " + std::to_string(P.vec_ok ? 1 : 0) +
         ", out_dtype = " + std::to_string(out_dtype) + ";\n";
    s += "    static constexpr unsigned char hcode[] = {" + byte_list(P.hcode, 2 * P.ninstr) + "};\n";
    s += "    static constexpr unsigned char leaf_dtype[] = {" + byte_list(ld, P.nleaves) + "};\n";
    s += "    static constexpr unsigned char leaf_scalar[] = {" + byte_list(ls, P.nleaves) + "};\n};\n}\n";
    if (red) {
        s += "extern \"C\" __global__ void __launch_bounds__(256) b200_jit_reduce_kernel(const __grid_constant__ b200::ProgramDesc P, "
             "const __grid_constant__ b200::LeafDesc O, const __grid_constant__ b200::GenericPlan G, void* partials, "
             "unsigned int* counters, b200::RedOut out) {\n    b200::grid_dependency_wait();\n    b200::grid_dependency_release();\n"
             "    b200::reduce_program_body<";
        s += C.wide ? "true" : "false";
        s += ", b200::StaticCode>(P, O, G, (b200::RawOf<";
        s += C.wide ? "true" : "false";
        s += ">::type*)partials, counters, out);\n}\n";
        return s;
    }
    s += "extern \"C\" __global__ void __launch_bounds__(256, 3) b200_jit_kernel(const __grid_constant__ b200::ProgramDesc P, "
         "const __grid_constant__ b200::LeafDesc O, long long n) {\n    b200::grid_dependency_wait();\n    b200::grid_dependency_release();\n"
         "    b200::ew_program_body<";
    s += C.wide ? "true" : "false";
    s += ", b200::StaticCode>(P, O, n);\n}\n";
    return s;
}

// Minimal stand-ins for the two C headers the sources include; NVRTC has no host library.
const char kStdint[] =
    "#pragma once\n"
    "typedef signed char int8_t; typedef short int16_t; typedef int int32_t; typedef long long int64_t;\n"
    "typedef unsigned char uint8_t; typedef unsigned short uint16_t; typedef unsigned int uint32_t; typedef unsigned long long uint64_t;\n"
    "typedef unsigned long uintptr_t;\n"
    "#ifndef UINT64_MAX\n#define UINT64_MAX 0xffffffffffffffffull\n#endif\n";
const char kStddef[] = "#pragma once\ntypedef unsigned long size_t;\n";

bool compile(const std::string& src, std::vector<char>* cubin) {
    if (!load_nvrtc()) { g_last_log = "libnvrtc could not be loaded"; return false; }
    const char* header_src[] = {kRtcProgram, kRtcCommon, kRtcReduce, kRtcHeader, kStdint, kStddef};
    const char* header_names[] = {"program.cuh", "common.cuh", "reduce_program.cuh", "../../include/b200arrays.h", "stdint.h", "stddef.h"};
    nvrtcProgram prog = nullptr;
    if (g_nvrtc.CreateProgram(&prog, src.c_str(), "b200_jit.cu", 6, header_src, header_names) != NVRTC_SUCCESS) return false;
    std::string inc = std::string("-I") + (getenv("B200_CUDA_INCLUDE") ? getenv("B200_CUDA_INCLUDE") : "/usr/local/cuda/include");
    // B200_LOG=debug: ptxas reports registers, spills and shared memory of every kernel it builds
    static const bool verbose = [] { const char* e = getenv("B200_LOG"); return e && strcmp(e, "debug") == 0; }();
    const char* opts[] = {"--gpu-architecture=sm_100a", "--std=c++17", "--fmad=false", inc.c_str(), "--ptxas-options=-v"};
    const nvrtcResult r = g_nvrtc.CompileProgram(prog, verbose ? 5 : 4, opts);
    bool ok = r == NVRTC_SUCCESS;
    if (ok && verbose) {
        size_t n = 0;
        std::string log;
        if (g_nvrtc.GetProgramLogSize(prog, &n) == NVRTC_SUCCESS && n > 1) {
            log.resize(n);
            g_nvrtc.GetProgramLog(prog, &log[0]);
            log_debug("run-time compiler: %.480s", log.c_str());
        }
    }
    if (!ok) {
        size_t n = 0;
        if (g_nvrtc.GetProgramLogSize(prog, &n) == NVRTC_SUCCESS && n > 1) {
            g_last_log.resize(n);
            g_nvrtc.GetProgramLog(prog, &g_last_log[0]);
        }
    } else {
        size_t n = 0;
        ok = g_nvrtc.GetCUBINSize(prog, &n) == NVRTC_SUCCESS && n > 0;
        if (ok) {
            cubin->resize(n);
            ok = g_nvrtc.GetCUBIN(prog, cubin->data()) == NVRTC_SUCCESS;
        }
    }
    g_nvrtc.DestroyProgram(&prog);
    return ok;
}

// Looks the expression up, compiling it on a miss.  Returns null when no specialised kernel exists.
Entry* lookup(const Compiled& C, int out_dtype, const ReduceInfo* red = nullptr) {
    const std::string key = cache_key(C, out_dtype, red);
    auto it = g_cache.find(key);
    if (it != g_cache.end()) {
        if (it->second.cubin.empty()) return nullptr;
        ++g_hits;
        return &it->second;
    }
    Entry e;
    if (compile(generate_source(C, out_dtype, red), &e.cubin)) ++g_compiled;
    else { ++g_failures; e.cubin.clear(); }
    Entry& slot = g_cache[key] = std::move(e);
    return slot.cubin.empty() ? nullptr : &slot;
}

}  // namespace

// Compiles (or finds) the specialised kernel without touching a device.  B200_OK when one exists.
int32_t jit_prepare(const Compiled& C, int out_dtype) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!enabled()) return fail(B200_UNSUPPORTED, "run-time specialisation is switched off");
    if (!lookup(C, out_dtype)) return fail(B200_UNSUPPORTED, "run-time specialisation failed: %.400s", g_last_log.c_str());
    return B200_OK;
}

// The same for the kernel of a mapreduce over this map expression.
int32_t jit_prepare_reduce(const Compiled& C, int out_dtype, int redop, int acc_dtype, int full) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!enabled()) return fail(B200_UNSUPPORTED, "run-time specialisation is switched off");
    const ReduceInfo red{redop, acc_dtype, full};
    if (!lookup(C, out_dtype, &red)) return fail(B200_UNSUPPORTED, "run-time specialisation failed: %.400s", g_last_log.c_str());
    return B200_OK;
}

// Launches the specialised kernel for this expression if there is one.  1: launched; 0: there is
// none, the caller interprets; -1: the kernel would have to be compiled or loaded now and the
// stream is being captured - the caller reports that the expression must run once outside a
// capture first (loading code is not something a capture can record).
static int acquire(b200_stream_t st, const Compiled& C, int out_dtype, const ReduceInfo* red, const char* symbol,
                   cudaKernel_t* kernel, int* per_sm) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!enabled()) return 0;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st->s, &cap) != cudaSuccess) { cudaGetLastError(); cap = cudaStreamCaptureStatusNone; }
    if (cap != cudaStreamCaptureStatusNone) {
        auto it = g_cache.find(cache_key(C, out_dtype, red));
        if (it == g_cache.end() || (!it->second.cubin.empty() && !it->second.kernel)) return -1;
    }
    Entry* e = lookup(C, out_dtype, red);
    if (!e) return 0;
    if (!e->kernel) {
        if (cudaLibraryLoadData(&e->lib, e->cubin.data(), nullptr, nullptr, 0, nullptr, nullptr, 0) != cudaSuccess ||
            cudaLibraryGetKernel(&e->kernel, e->lib, symbol) != cudaSuccess) {
            cudaGetLastError();
            ++g_failures;
            e->cubin.clear();
            e->kernel = nullptr;
            return 0;
        }
        int b = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&b, (const void*)e->kernel, 256, 0) != cudaSuccess || b < 1) {
            cudaGetLastError();
            b = 3;
        }
        e->blocks_per_sm = b;
    }
    *kernel = e->kernel;
    *per_sm = e->blocks_per_sm;
    return 1;
}

int jit_broadcast(b200_stream_t st, const Compiled& C, const LeafDesc& O, int64_t n) {
    cudaKernel_t kernel = nullptr;
    int per_sm = 0;
    const int got = acquire(st, C, O.dtype, nullptr, "b200_jit_kernel", &kernel, &per_sm);
    if (got <= 0) return got;
    const int64_t nvec = (n + kVec - 1) / kVec;
    // one vector per thread and the hardware block scheduler rather than a persistent wave
    // (measured on B200 at 2^26 elements: 151 / 150 / 156 us against 155 / 160 / 208 us for the
    // three benchmark trees); the kernel's grid-stride loop covers what the cap leaves over
    (void)per_sm;
    int64_t blocks = (nvec + 255) / 256;
    if (blocks < 1) blocks = 1;
    if (blocks > 0x7fffffff) blocks = 0x7fffffff;
    const unsigned grid = (unsigned)blocks;
    long long nn = n;
    void* args[] = {(void*)&C.P, (void*)&O, (void*)&nn};
    if (launch_overlapped_handle((const void*)kernel, grid, 256, args, st->s) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return 1;
}

// The specialised kernel for mapreducedim! over this map expression: same return values as
// jit_broadcast; on 1, *kernel takes (ProgramDesc, LeafDesc, GenericPlan, partials, counters,
// RedOut) like reduce_program_kernel and *resident is one wave of its blocks on this device.
int jit_reduce_kernel(b200_stream_t st, const Compiled& C, int out_dtype, int redop, int acc_dtype, int full,
                      const void** kernel, int64_t* resident) {
    const ReduceInfo red{redop, acc_dtype, full};
    cudaKernel_t k = nullptr;
    int per_sm = 0;
    const int got = acquire(st, C, out_dtype, &red, "b200_jit_reduce_kernel", &k, &per_sm);
    if (got <= 0) return got;
    *kernel = (const void*)k;
    *resident = (int64_t)per_sm * sm_count(st->dev);
    return 1;
}

}  // namespace b200

using namespace b200;

extern "C" int32_t b200_jit_configure(int32_t enable) {
    std::lock_guard<std::mutex> lk(g_mu);
    g_enabled = enable ? 1 : 0;
    return B200_OK;
}

extern "C" int32_t b200_jit_stats(uint64_t out[4]) {
    if (!out) return fail(B200_INVALID_ARG, "null output");
    std::lock_guard<std::mutex> lk(g_mu);
    out[0] = g_compiled;
    out[1] = g_hits;
    out[2] = g_failures;
    out[3] = enabled() ? 1 : 0;
    return B200_OK;
}
