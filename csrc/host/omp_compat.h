// OpenMP when the translation unit is built with -fopenmp, single-threaded
// stand-ins otherwise (the ThreadSanitizer build: libgomp is not instrumented,
// so its barriers would be reported as races).
#pragma once
#ifdef _OPENMP
#include <omp.h>
#else
static inline int omp_get_max_threads() { return 1; }
static inline int omp_get_thread_num() { return 0; }
#endif
