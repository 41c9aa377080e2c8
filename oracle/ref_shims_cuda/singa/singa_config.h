// Stand-in for the singa_config.h apache/singa's CMake generates
// (cmake/Templates/singa_config.h.in): the CUDA + cuDNN + distributed (NCCL)
// configuration, without DNNL, OpenCL or glog.  TEST INFRASTRUCTURE ONLY.
#ifndef SINGA_CONFIG_H_
#define SINGA_CONFIG_H_
#define USE_CBLAS
#define USE_CUDA
#define USE_CUDNN
#define USE_DIST
#define SINGA_MAJOR_VERSION 5
#define SINGA_MINOR_VERSION 1
#define SINGA_PATCH_VERSION 0
#define SINGA_VERSION 5100
#endif
