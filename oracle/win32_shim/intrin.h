/* intrin.h — stand-in for the MSVC header of that name; gcc's <cpuid.h>/<immintrin.h>
 * (pulled in by the windows.h stand-in beside this file) already provide __cpuidex and
 * _xgetbv. TEST INFRASTRUCTURE ONLY. */
#ifndef SP_ORACLE_INTRIN_SHIM_H
#define SP_ORACLE_INTRIN_SHIM_H
#include <cpuid.h>
#include <immintrin.h>
#endif
