// Multi-tensor kernels: one launch covers a whole list of parameter tensors.
//   * fused SGD update (weight decay, momentum, dampening, Nesterov, 1/world
//     gradient scaling) - one pass over p, g, m instead of the reference's
//     chain of 8-10 BLAS-1 / elementwise launches per tensor;
//   * bucket pack / unpack between a list of gradient tensors and the
//     communicator's flat staging buffer, with the fp32->fp16 cast on the way
//     in and the fp16->fp32 cast (+ scale) on the way out.
// The tensor table (pointers, sizes, first-tile index) travels in the kernel
// argument buffer, so there is no host-to-device table copy and no
// allocation; lists longer than kMaxTensors are split into several launches.
// Every CTA handles one 1024-element tile and finds its tensor with a binary
// search over the table.
#include "common.cuh"

namespace sgb {
namespace {

constexpr int kBlock = 256;
constexpr int kTile = 1024;       // elements per CTA (one float4 per thread)
constexpr int kMaxTensors = 72;   // 72 * 40 B + header < 4 KB of kernel arguments

struct Table {
  int count;
  unsigned first_tile[kMaxTensors + 1];
  unsigned long long n[kMaxTensors];
  void* a[kMaxTensors];  // param            | packed tensor
  void* b[kMaxTensors];  // grad             | (unused)
  void* c[kMaxTensors];  // momentum buffer  | (unused)
};
// flat-buffer element offset of tensor k (pack / unpack)
struct Offsets {
  unsigned long long off[kMaxTensors];
};

__device__ __forceinline__ int find_tensor(const Table& t, unsigned tile) {
  int lo = 0, hi = t.count - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (t.first_tile[mid] <= tile) lo = mid; else hi = mid - 1;
  }
  return lo;
}

struct SgdArgs {
  float lr, mom, damp, decay, grad_scale;
  int use_momentum, nesterov, use_decay, use_scale;
};

__device__ __forceinline__ void sgd_one(float& p, float g, float& m, const SgdArgs& a) {
  // the reference's chain, one rounding per BLAS-1 step (python/singa/opt.py):
  //   g *= 1/world ; g += decay*p ; m = m*mom ; m += (1-damp)*g ; p += -lr*m
  if (a.use_scale) g = g * a.grad_scale;
  if (a.use_decay) g = fmaf(a.decay, p, g);
  float step = g;
  if (a.use_momentum) {
    float b = m * a.mom;
    b = fmaf(1.0f - a.damp, g, b);
    m = b;
    step = a.nesterov ? fmaf(a.mom, b, g) : b;
  }
  p = fmaf(0.0f - a.lr, step, p);
}

__global__ void __launch_bounds__(kBlock)
sgd_multi_kernel(const __grid_constant__ Table t, const SgdArgs a) {
  const int k = find_tensor(t, blockIdx.x);
  const size_t n = t.n[k];
  const size_t base = static_cast<size_t>(blockIdx.x - t.first_tile[k]) * kTile;
  float* p = static_cast<float*>(t.a[k]);
  const float* g = static_cast<const float*>(t.b[k]);
  float* m = static_cast<float*>(t.c[k]);
  const bool vec = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) |
                     (a.use_momentum ? reinterpret_cast<uintptr_t>(m) : 0)) & 15u) == 0;
  const size_t i = base + 4 * threadIdx.x;
  if (vec && i + 4 <= n) {
    Vec4f vp, vg, vm;
    vp.u = ld128(p + i);
    vg.u = ld128(g + i);
    if (a.use_momentum) vm.u = ld128(m + i);
#pragma unroll
    for (int j = 0; j < 4; ++j) sgd_one(vp.f[j], vg.f[j], vm.f[j], a);
    st128(p + i, vp.u);
    if (a.use_momentum) st128(m + i, vm.u);
  } else {
    for (size_t j = i; j < n && j < i + 4; ++j) {
      float pv = p[j], mv = a.use_momentum ? m[j] : 0.f;
      sgd_one(pv, g[j], mv, a);
      p[j] = pv;
      if (a.use_momentum) m[j] = mv;
    }
  }
}

enum PackMode { kPackF32 = 0, kPackF32ToF16 = 1, kUnpackF32 = 2, kUnpackF16ToF32 = 3 };

template <int MODE>
__global__ void __launch_bounds__(kBlock)
pack_multi_kernel(const __grid_constant__ Table t, const __grid_constant__ Offsets o,
                  void* flat, float scale, int use_scale) {
  const int k = find_tensor(t, blockIdx.x);
  const size_t n = t.n[k];
  const size_t i = static_cast<size_t>(blockIdx.x - t.first_tile[k]) * kTile + 4 * threadIdx.x;
  if (i >= n) return;
  float* tensor = static_cast<float*>(t.a[k]);
  const size_t fo = o.off[k] + i;
  const bool full = i + 4 <= n;
  if (MODE == kPackF32 || MODE == kUnpackF32) {
    float* fl = static_cast<float*>(flat) + fo;
    const bool vec = full && ((reinterpret_cast<uintptr_t>(tensor + i) |
                               reinterpret_cast<uintptr_t>(fl)) & 15u) == 0;
    if (MODE == kPackF32) {
      if (vec) st128(fl, ld128(tensor + i));
      else for (size_t j = 0; j < 4 && i + j < n; ++j) fl[j] = tensor[i + j];
    } else {
      if (vec) {
        Vec4f v; v.u = ld128(fl);
        if (use_scale) {
#pragma unroll
          for (int j = 0; j < 4; ++j) v.f[j] = v.f[j] * scale;
        }
        st128(tensor + i, v.u);
      } else {
        for (size_t j = 0; j < 4 && i + j < n; ++j)
          tensor[i + j] = use_scale ? fl[j] * scale : fl[j];
      }
    }
  } else {
    __half* fl = static_cast<__half*>(flat) + fo;
    const bool vec = full && (reinterpret_cast<uintptr_t>(tensor + i) & 15u) == 0 &&
                     (reinterpret_cast<uintptr_t>(fl) & 7u) == 0;
    if (MODE == kPackF32ToF16) {
      if (vec) {
        Vec4f v; v.u = ld128(tensor + i);
        union { uint2 u; __half h[4]; } h;
#pragma unroll
        for (int j = 0; j < 4; ++j) h.h[j] = __float2half_rn(v.f[j]);
        *reinterpret_cast<uint2*>(fl) = h.u;
      } else {
        for (size_t j = 0; j < 4 && i + j < n; ++j) fl[j] = __float2half_rn(tensor[i + j]);
      }
    } else {
      if (vec) {
        union { uint2 u; __half h[4]; } h;
        h.u = *reinterpret_cast<const uint2*>(fl);
        Vec4f v;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float f = __half2float(h.h[j]);
          v.f[j] = use_scale ? f * scale : f;
        }
        st128(tensor + i, v.u);
      } else {
        for (size_t j = 0; j < 4 && i + j < n; ++j) {
          const float f = __half2float(fl[j]);
          tensor[i + j] = use_scale ? f * scale : f;
        }
      }
    }
  }
}

// Fills a table with tensors [first, first+count) and returns the tile count.
unsigned fill_table(Table& t, Offsets* o, void* const* a, void* const* b, void* const* c,
                    const size_t* sizes, size_t first, int count, size_t flat_off0) {
  t.count = count;
  unsigned tiles = 0;
  size_t off = flat_off0;
  for (int k = 0; k < count; ++k) {
    t.first_tile[k] = tiles;
    t.n[k] = sizes[first + k];
    t.a[k] = a[first + k];
    t.b[k] = b ? b[first + k] : nullptr;
    t.c[k] = c ? c[first + k] : nullptr;
    if (o) o->off[k] = off;
    off += sizes[first + k];
    tiles += static_cast<unsigned>(ceil_div(sizes[first + k], kTile));
  }
  t.first_tile[count] = tiles;
  return tiles;
}

int pack_common(int mode, void* const* tensors, const size_t* sizes, size_t count, void* flat,
                size_t flat_offset, float scale, int use_scale, void* stream) {
  if (count == 0) return SGB_OK;
  if (!tensors || !sizes || !flat) return SGB_ERR_NULL;
  cudaStream_t s = as_stream(stream);
  size_t off = flat_offset;
  for (size_t first = 0; first < count;) {
    // take as many tensors as fit the table, skipping empty ones
    Table t;
    Offsets o;
    void* ptrs[kMaxTensors];
    size_t ns[kMaxTensors];
    int cnt = 0;
    size_t chunk_off = off;
    unsigned long long tiles64 = 0;
    while (first < count && cnt < kMaxTensors) {
      const size_t n = sizes[first];
      if (n && !tensors[first]) return SGB_ERR_NULL;
      const unsigned long long tl = ceil_div(n, kTile);
      if (tiles64 + tl > 0x7fffffffull) {
        if (cnt == 0) return SGB_ERR_SIZE;
        break;
      }
      if (n) {
        // empty tensors keep their place in the flat buffer (0 elements)
        ptrs[cnt] = tensors[first];
        ns[cnt] = n;
        if (cnt == 0) chunk_off = off;
        ++cnt;
        tiles64 += tl;
      }
      off += n;
      ++first;
      if (n == 0) continue;
    }
    if (cnt == 0) continue;
    // offsets inside the chunk are contiguous because empty tensors add 0
    const unsigned tiles = fill_table(t, &o, ptrs, nullptr, nullptr, ns, 0, cnt, chunk_off);
    switch (mode) {
      case kPackF32: pack_multi_kernel<kPackF32><<<tiles, kBlock, 0, s>>>(t, o, flat, scale, use_scale); break;
      case kPackF32ToF16: pack_multi_kernel<kPackF32ToF16><<<tiles, kBlock, 0, s>>>(t, o, flat, scale, use_scale); break;
      case kUnpackF32: pack_multi_kernel<kUnpackF32><<<tiles, kBlock, 0, s>>>(t, o, flat, scale, use_scale); break;
      default: pack_multi_kernel<kUnpackF16ToF32><<<tiles, kBlock, 0, s>>>(t, o, flat, scale, use_scale); break;
    }
  }
  return launch_status();
}

}  // namespace
}  // namespace sgb

using namespace sgb;

extern "C" {

int sgb_sgd_update_multi_f32(void* const* params, void* const* grads, void* const* moments,
                             const size_t* sizes, size_t count, float lr, float momentum,
                             float dampening, float weight_decay, int nesterov, float grad_scale,
                             void* stream) {
  if (count == 0) return SGB_OK;
  if (!params || !grads || !sizes) return SGB_ERR_NULL;
  const int use_m = momentum != 0.0f;
  if (use_m && !moments) return SGB_ERR_NULL;
  if (nesterov && (!use_m || dampening != 0.0f)) return SGB_ERR_UNSUPPORTED;
  SgdArgs a{lr, momentum, dampening, weight_decay, grad_scale, use_m, nesterov != 0,
            weight_decay != 0.0f, grad_scale != 1.0f};
  cudaStream_t s = as_stream(stream);
  for (size_t first = 0; first < count;) {
    Table t;
    void *pa[kMaxTensors], *pb[kMaxTensors], *pc[kMaxTensors];
    size_t ns[kMaxTensors];
    int cnt = 0;
    unsigned long long tiles64 = 0;
    while (first < count && cnt < kMaxTensors) {
      const size_t n = sizes[first];
      if (n) {
        if (!params[first] || !grads[first] || (use_m && !moments[first])) return SGB_ERR_NULL;
        const unsigned long long tl = ceil_div(n, kTile);
        if (tiles64 + tl > 0x7fffffffull) {
          if (cnt == 0) return SGB_ERR_SIZE;
          break;
        }
        pa[cnt] = params[first];
        pb[cnt] = grads[first];
        pc[cnt] = use_m ? moments[first] : nullptr;
        ns[cnt] = n;
        ++cnt;
        tiles64 += tl;
      }
      ++first;
    }
    if (cnt == 0) continue;
    const unsigned tiles = fill_table(t, nullptr, pa, pb, pc, ns, 0, cnt, 0);
    sgd_multi_kernel<<<tiles, kBlock, 0, s>>>(t, a);
  }
  return launch_status();
}

int sgb_sgd_update_f32(float* param, const float* grad, float* moment, size_t n, float lr,
                       float momentum, float dampening, float weight_decay, int nesterov,
                       float grad_scale, void* stream) {
  void* p[1] = {param};
  void* g[1] = {const_cast<float*>(grad)};
  void* m[1] = {moment};
  size_t ns[1] = {n};
  return sgb_sgd_update_multi_f32(p, g, m, ns, 1, lr, momentum, dampening, weight_decay,
                                  nesterov, grad_scale, stream);
}

int sgb_pack_f32(void* const* tensors, const size_t* sizes, size_t count, float* flat,
                 size_t flat_offset, void* stream) {
  return pack_common(kPackF32, tensors, sizes, count, flat, flat_offset, 1.f, 0, stream);
}
int sgb_pack_f32_to_f16(void* const* tensors, const size_t* sizes, size_t count, void* flat_f16,
                        size_t flat_offset, void* stream) {
  return pack_common(kPackF32ToF16, tensors, sizes, count, flat_f16, flat_offset, 1.f, 0, stream);
}
int sgb_unpack_f32(const float* flat, size_t flat_offset, void* const* tensors,
                   const size_t* sizes, size_t count, float scale, void* stream) {
  return pack_common(kUnpackF32, tensors, sizes, count, const_cast<float*>(flat), flat_offset,
                     scale, scale != 1.0f, stream);
}
int sgb_unpack_f16_to_f32(const void* flat_f16, size_t flat_offset, void* const* tensors,
                          const size_t* sizes, size_t count, float scale, void* stream) {
  return pack_common(kUnpackF16ToF32, tensors, sizes, count, const_cast<void*>(flat_f16),
                     flat_offset, scale, scale != 1.0f, stream);
}

}  // extern "C"
