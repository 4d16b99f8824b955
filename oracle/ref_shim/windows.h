/* Empty stand-in: the reference includes <windows.h> unconditionally
 * (srcs/core/include.h:24) but the GEMM path uses nothing from it. */
