// Stand-in for the singa_config.h that apache/singa's CMake generates from
// cmake/Templates/singa_config.h.in: the CPU-only configuration with a CBLAS
// (no CUDA, no DNNL, no glog, no distributed support).  TEST INFRASTRUCTURE.
#ifndef SINGA_CONFIG_H_
#define SINGA_CONFIG_H_
#define CPU_ONLY
#define USE_CBLAS
#define SINGA_MAJOR_VERSION 5
#define SINGA_MINOR_VERSION 1
#define SINGA_PATCH_VERSION 0
#define SINGA_VERSION 5100
#endif
