/*
 * ref_cpu_gemm.cpp -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * Command-line driver around the reference's OWN CPU GEMM,
 * decx::sgemm_caller<TX,TY> (srcs/GEMM/CPU/sgemm_callers.h:1227-1249), compiled
 * from the reference tree where it lies (the include path is given by the
 * Makefile; no reference source is copied).  Used to pin the oracle's fmaf
 * chain and as the timed CPU baseline.
 *
 * What the shim below supplies, and why:
 *  - `windows.h`: an empty header on the include path (core/include.h:24).
 *  - `__m256` wrapper: the reference reads lanes as `v.m256_f32[i]`
 *    (sgemm_calc_kernel.h:27-28,34), a member MSVC's __m256 union has and
 *    GCC's vector type has not.  A union with the same member and implicit
 *    conversions makes the reference source compile untouched.
 *  - `_DECX_CPU_CODES_`, `__align__`, `__int64`, console-colour macros: what
 *    the MSVC project defines (thread_pool.h:251-253, decx_utils_macros.h:96-98,
 *    vector_defines.h:57, error.h:17-21).
 *
 * The reference's global thread pool starts hardware_concurrency() workers
 * at static-initialisation time into arrays of 16 slots (thread_pool.h:18,
 * 141-150, 246); this program caps that count itself (see get_nprocs below).
 *
 * Usage: decx_ref_cpu gemm M N K TXxTY reps A B Cout
 *   A, B: "seed:<n>" (seeded uniform [-1,1), same generator as the oracle) or a
 *   raw little-endian float32 file, row-major, row stride = width.
 *   Cout: "-" or a file that receives the M*N result.
 * Prints one JSON line {"best_s":..,"median_s":..,"gflops":..,"threads":..}.
 */
#include <immintrin.h>
#include <mutex>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <cstdint>
#include <chrono>
#include <vector>
#include <algorithm>
#include <string>

/* The reference's global pool is built during static initialisation with
 * std::thread::hardware_concurrency() workers placed into arrays of 16 slots
 * (thread_pool.h:18, :144-150, :246).  With glibc >= 2.35 that count is the number of CPUs the
 * machine has online, not the size of the affinity mask, so on a host with more than 16 CPUs
 * the pool overruns its arrays whatever `taskset` says (seen as an abort inside
 * pthread_mutex_lock on 24-CPU hosts).  Two measures, both taken before the pool exists:
 *   - get_nprocs(), which the C++ runtime asks for that count, is defined here and answers
 *     with the CPUs this process may use, at most 16 (or DECX_REF_CPUS);
 *   - the affinity mask is narrowed to the same CPUs, so the workers do not migrate.
 * The guard object is defined before the reference headers are included, so it is constructed
 * first. */
#include <sched.h>
#include <unistd.h>
static int g_pool_cpus = 0;
static int usable_cpus(cpu_set_t* want)
{
    cpu_set_t have;
    if (want) CPU_ZERO(want);
    if (sched_getaffinity(0, sizeof have, &have) != 0) return 1;
    int limit = 16;
    if (const char* e = getenv("DECX_REF_CPUS")) { int v = atoi(e); if (v >= 1 && v <= 16) limit = v; }
    int n = 0;
    for (int c = 0; c < CPU_SETSIZE && n < limit; ++c)
        if (CPU_ISSET(c, &have)) { if (want) CPU_SET(c, want); ++n; }
    return n > 0 ? n : 1;
}
extern "C" int get_nprocs(void)
{
    return g_pool_cpus > 0 ? g_pool_cpus : usable_cpus(nullptr);
}
struct AffinityGuard {
    AffinityGuard()
    {
        cpu_set_t want;
        int n = usable_cpus(&want);
        if (CPU_COUNT(&want) > 0) sched_setaffinity(0, sizeof want, &want);
        g_pool_cpus = n;
    }
};
static AffinityGuard g_affinity_guard;

struct decx_shim_m256 {
    union { __m256 v; float m256_f32[8]; };
    decx_shim_m256() {}
    decx_shim_m256(__m256 x) : v(x) {}
    operator __m256() const { return v; }
};

#define _DECX_CPU_CODES_
#define __align__(n) __attribute__((aligned(n)))
#define __int64 long long
#define SetConsoleColor(x) ((void)0)
#define ResetConsoleColor ((void)0)
#define __m256 decx_shim_m256
#include "GEMM/CPU/sgemm_callers.h"
#undef __m256

extern "C" void decxo_fill_uniform(float* dst, uint64_t n, uint32_t seed, uint64_t first_index);

static float* alloc_f(size_t n)
{
    void* p = nullptr;
    if (posix_memalign(&p, 64, (n * sizeof(float) + 63) / 64 * 64 + 4096)) return nullptr;
    memset(p, 0, (n * sizeof(float) + 63) / 64 * 64 + 4096);
    return (float*)p;
}

static bool load(const char* spec, float* dst, size_t n)
{
    if (!strncmp(spec, "seed:", 5)) { decxo_fill_uniform(dst, n, (uint32_t)atoi(spec + 5), 0); return true; }
    FILE* f = fopen(spec, "rb");
    if (!f) return false;
    size_t got = fread(dst, sizeof(float), n, f);
    fclose(f);
    return got == n;
}

typedef void (*caller_t)(float*, float*, float*, float*, const int4*);

static caller_t pick(int tx, int ty)
{
    if (tx == 1 && ty == 1) return decx::sgemm_caller<1, 1>;
    if (tx == 2 && ty == 2) return decx::sgemm_caller<2, 2>;
    if (tx == 4 && ty == 2) return decx::sgemm_caller<4, 2>;
    if (tx == 3 && ty == 4) return decx::sgemm_caller<3, 4>;   /* the shipped instantiation, sgemm.h:54 */
    if (tx == 4 && ty == 4) return decx::sgemm_caller<4, 4>;
    return nullptr;
}

int main(int argc, char** argv)
{
    if (argc < 10 || strcmp(argv[1], "gemm")) {
        fprintf(stderr, "usage: %s gemm M N K TXxTY reps A B Cout\n", argv[0]);
        return 2;
    }
    const long M = atol(argv[2]), N = atol(argv[3]), K = atol(argv[4]);
    int tx = 0, ty = 0;
    if (sscanf(argv[5], "%dx%d", &tx, &ty) != 2) return 2;
    const int reps = atoi(argv[6]);
    caller_t fn = pick(tx, ty);
    /* more tasks than workers makes the reference's queue picker index queues that were never
     * constructed (thread_pool.h:72-99 returns a queue LENGTH as an index) */
    if (g_pool_cpus > 0 && tx * ty > g_pool_cpus) {
        fprintf(stderr, "thread split %dx%d needs %d CPUs, %d available\n", tx, ty, tx * ty, g_pool_cpus);
        return 7;
    }
    /* Preconditions of the reference entry (sgemm_callers.h:231,307,1120,1231-1248;
     * aligned loads sgemm_calc_kernel.h:207-211): */
    if (!fn || K % 8 || N % 8 || K < 64 || (M / tx) % 32 || (M % tx) || (N / 16) / ty < 1) {
        fprintf(stderr, "shape/thread split outside what the reference entry supports\n");
        return 3;
    }
    float* A = alloc_f((size_t)M * K); float* B = alloc_f((size_t)K * N);
    float* T = alloc_f((size_t)K * N); float* C = alloc_f((size_t)M * N);
    if (!A || !B || !T || !C) return 4;
    if (!load(argv[7], A, (size_t)M * K) || !load(argv[8], B, (size_t)K * N)) { fprintf(stderr, "bad input\n"); return 5; }
    int4 dims; dims.x = (int)K; dims.y = (int)M; dims.z = (int)N; dims.w = 0;
    std::vector<double> t;
    for (int r = 0; r < reps; ++r) {
        auto t0 = std::chrono::steady_clock::now();
        fn(A, B, T, C, &dims);
        auto t1 = std::chrono::steady_clock::now();
        t.push_back(std::chrono::duration<double>(t1 - t0).count());
    }
    if (strcmp(argv[9], "-")) {
        FILE* f = fopen(argv[9], "wb");
        if (!f || fwrite(C, sizeof(float), (size_t)M * N, f) != (size_t)M * N) return 6;
        fclose(f);
    }
    std::sort(t.begin(), t.end());
    printf("{\"best_s\": %.9f, \"median_s\": %.9f, \"gflops\": %.3f, \"threads\": %d, \"reps\": %d}\n",
           t.front(), t[t.size() / 2], 2.0 * M * N * K / t.front() / 1e9, tx * ty, reps);
    fflush(stdout);
    _Exit(0);   /* skip static destructors: the pool's workers never join */
}
