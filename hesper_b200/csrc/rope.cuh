// rope.cuh -- NeoX RoPE + f16 KV-cache write for one (token, head, pair) element; shared by
// the stand-alone kernel and by the q/k/v matvec kernel that runs it as its tail.
#pragma once

#include "common.cuh"

namespace hb {

struct RopeParams {
  float* q;          // [B][H][D] rotated in place
  const float* k;    // [B][Hkv][D]
  const float* v;    // [B][Hkv][D]
  __half* k_cache;   // [B/T][Hkv][slots][D]
  __half* v_cache;
  const int32_t* pos;  // [B/T] position of each sequence's first new token
  int B, H, Hkv, D, slots, ring;
  int T;               // new tokens per sequence (1 = decode); B counts tokens
  double base;
  const double2* table;  // nullable [B][D/2] (cos, sin) of every token's angles, see rope_angle
};

// theta = pos * base^(-2i/D).  The angle reaches thousands of radians, where f32 loses four
// digits: the few thousand rotations of a step are done in double.
__device__ __forceinline__ double2 rope_angle(int pos, int i, int D, double base) {
  const double theta = (double)pos * pow(base, -2.0 * (double)i / (double)D);
  double sn, cs;
  sincos(theta, &sn, &cs);
  return make_double2(cs, sn);
}

// Element idx of B * (H + 2*Hkv) * D/2: heads 0..H-1 are Q heads (rotated in place), H..H+Hkv-1
// K heads (rotated, then written to the cache as f16), the rest V rows (packed alongside).
// COHERENT: read q/k/v through L2 (the caller's own grid wrote them moments ago).
template <bool COHERENT>
__device__ __forceinline__ void rope_kv_element(const RopeParams& p, long idx) {
  auto ld = [](const float* a) { return COHERENT ? __ldcg(a) : *a; };
  const int half = p.D >> 1;
  const int per_seq = (p.H + 2 * p.Hkv) * half;
  const int b = (int)(idx / per_seq);
  const int r = (int)(idx % per_seq);
  const int head = r / half, i = r % half;
  const int cb = b / p.T;  // which sequence's cache
  const int pos = p.pos[cb] + (b - cb * p.T);
  int slot = p.ring ? pos % p.slots : pos;
  slot = slot < 0 ? 0 : (slot >= p.slots ? p.slots - 1 : slot);
  if (head < p.H + p.Hkv) {
    // the angles are the same in every layer of a step: a caller that runs many layers
    // computes them once into `table`
    const double2 a = p.table ? p.table[(size_t)b * half + i] : rope_angle(pos, i, p.D, p.base);
    const double cs = a.x, sn = a.y;
    if (head < p.H) {
      float* qh = p.q + ((size_t)b * p.H + head) * p.D;
      const double x0 = ld(qh + i), x1 = ld(qh + i + half);
      qh[i] = (float)(x0 * cs - x1 * sn);
      qh[i + half] = (float)(x0 * sn + x1 * cs);
    } else {
      const int kh = head - p.H;
      const float* kk = p.k + ((size_t)b * p.Hkv + kh) * p.D;
      const double x0 = ld(kk + i), x1 = ld(kk + i + half);
      __half* dst = p.k_cache + (((size_t)cb * p.Hkv + kh) * p.slots + slot) * p.D;
      dst[i] = __float2half_rn((float)(x0 * cs - x1 * sn));
      dst[i + half] = __float2half_rn((float)(x0 * sn + x1 * cs));
    }
  } else {
    const int vh = head - p.H - p.Hkv;
    const float* vv = p.v + ((size_t)b * p.Hkv + vh) * p.D;
    __half* dst = p.v_cache + (((size_t)cb * p.Hkv + vh) * p.slots + slot) * p.D;
    dst[i] = __float2half_rn(ld(vv + i));
    dst[i + half] = __float2half_rn(ld(vv + i + half));
  }
}

}  // namespace hb
