// Point location on the icosphere hierarchy: for every (lon, lat) sample the face of the
// order-N mesh that the sample's ray from the origin hits, the three vertices of that face and
// the barycentric weights of the hit point.  This is what turns a gnomonic kernel or an image grid
// into a weighted (P = 3) sample map on mesh vertices.
//
// One thread per sample walks the hierarchy: a breadth-first search over the 20 faces of level 0,
// then on every finer level a search that starts at the centre child (4 f + 3) of the face found
// on the level above and spreads over neighbouring faces - almost always one to four tests.
// Same search order, acceptance test (barycentric coordinates >= -1e-3) and float32 arithmetic as
// the reference's host code (src/util/cpp/sphere.cpp:1007-1105, :1116-1270), which walks the same
// hierarchy with an OpenMP loop over samples and std::set / std::queue per sample; products and
// sums use the round-to-nearest intrinsics so that they are not contracted into FMAs.
#include "common.cuh"

namespace mc {

constexpr int SPHERE_MAX_LEVELS = 12;
constexpr int SPHERE_QUEUE = 96;  // faces one search may enqueue (level 0 has 20 in all)

struct SphereLevels {
  const float* v[SPHERE_MAX_LEVELS];    // (V_l, 3) vertex coordinates
  const int* fv[SPHERE_MAX_LEVELS];     // (F_l, 3) vertices of every face in half-edge walk order
  const int* fadj[SPHERE_MAX_LEVELS];   // (F_l, 3) faces across the three half-edges
  int nf[SPHERE_MAX_LEVELS];
};

struct V3 {
  float x, y, z;
};
__device__ __forceinline__ V3 ld3(const float* p, int i) {
  return {__ldg(p + 3 * i), __ldg(p + 3 * i + 1), __ldg(p + 3 * i + 2)};
}
__device__ __forceinline__ V3 sub(V3 a, V3 b) {
  return {__fsub_rn(a.x, b.x), __fsub_rn(a.y, b.y), __fsub_rn(a.z, b.z)};
}
__device__ __forceinline__ V3 scale(V3 a, float s) {
  return {__fmul_rn(a.x, s), __fmul_rn(a.y, s), __fmul_rn(a.z, s)};
}
__device__ __forceinline__ float dot(V3 a, V3 b) {
  return __fadd_rn(__fadd_rn(__fmul_rn(a.x, b.x), __fmul_rn(a.y, b.y)), __fmul_rn(a.z, b.z));
}
__device__ __forceinline__ V3 cross(V3 a, V3 b) {
  return {__fsub_rn(__fmul_rn(a.y, b.z), __fmul_rn(a.z, b.y)),
          __fsub_rn(__fmul_rn(a.z, b.x), __fmul_rn(a.x, b.z)),
          __fsub_rn(__fmul_rn(a.x, b.y), __fmul_rn(a.y, b.x))};
}
__device__ __forceinline__ V3 unit(V3 a) {
  const float n = __fsqrt_rn(dot(a, a));
  return {__fdiv_rn(a.x, n), __fdiv_rn(a.y, n), __fdiv_rn(a.z, n)};
}

// sphere.cpp:1055-1105: is the ray through pt inside face f (with a 1e-3 margin)?  s, t, u are the
// barycentric weights of walk vertices 2, 1, 0.
__device__ bool point_in_face(const SphereLevels& L, int lvl, int f, V3 pt, float& s, float& t,
                              float& u) {
  const int* fv = L.fv[lvl] + 3 * f;
  const V3 A = ld3(L.v[lvl], __ldg(fv)), B = ld3(L.v[lvl], __ldg(fv + 1)), C = ld3(L.v[lvl], __ldg(fv + 2));
  const V3 normal = unit(cross(sub(C, B), sub(A, B)));
  const float d = -dot(normal, A);
  const V3 ray = unit(pt);
  const float denom = dot(normal, ray);
  if (denom < 0.f) return false;  // a face on the far side of the sphere
  V3 proj;
  if ((double)denom < 1e-12) {
    const float dist = __fadd_rn(dot(normal, pt), d);
    proj = sub(pt, scale(normal, dist));
  } else {
    const float dist = __fdiv_rn(dot(A, normal), denom);
    proj = scale(ray, dist);
  }
  const V3 BA = sub(B, A), CA = sub(C, A);
  const V3 N = cross(BA, CA), W = sub(proj, A);
  const float nn = dot(N, N);
  s = __fdiv_rn(dot(cross(BA, W), N), nn);
  t = __fdiv_rn(dot(cross(W, CA), N), nn);
  u = __fsub_rn(__fsub_rn(1.f, s), t);
  return (double)s >= -1e-3 && (double)t >= -1e-3 && (double)u >= -1e-3;
}

// sphere.cpp:1007-1053: first face in breadth-first order from `start` that contains the point
// (-1 if the search runs out).
__device__ int search_faces(const SphereLevels& L, int lvl, int start, V3 pt, float& s, float& t,
                            float& u) {
  int queue[SPHERE_QUEUE];
  int head = 0, tail = 0;
  queue[tail++] = start;
  while (head < tail) {
    const int f = queue[head++];
    if (point_in_face(L, lvl, f, pt, s, t, u)) return f;
    for (int j = 0; j < 3; ++j) {
      const int a = __ldg(L.fadj[lvl] + 3 * f + j);
      bool seen = false;
      for (int q = 0; q < tail; ++q) seen |= queue[q] == a;
      if (!seen && tail < SPHERE_QUEUE) queue[tail++] = a;
    }
  }
  return -1;
}

__global__ void sphere_locate_kernel(const float* __restrict__ samples, long n, int order,
                                     SphereLevels L, int nearest, int64_t* __restrict__ face_idx,
                                     int64_t* __restrict__ vertex_idx, float* __restrict__ weights) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const float lon = __ldg(samples + 2 * i), lat = __ldg(samples + 2 * i + 1);
    // core/conversions.h:21-27
    const V3 pt = {__fmul_rn(cosf(lat), sinf(lon)), -sinf(lat), __fmul_rn(cosf(lat), cosf(lon))};
    float s = 0.f, t = 0.f, u = 0.f;
    int f = search_faces(L, 0, 0, pt, s, t, u);
    for (int lvl = 1; lvl <= order && f >= 0; ++lvl) {
      int start = 4 * f + 3;
      if (start >= L.nf[lvl]) start = L.nf[lvl] - 1;
      f = search_faces(L, lvl, start, pt, s, t, u);
    }
    face_idx[i] = f;
    if (f < 0) {  // (the reference leaves an out-of-range marker; nothing on a closed mesh gets here)
      for (int j = 0; j < 3; ++j) { vertex_idx[3 * i + j] = 0; weights[3 * i + j] = 0.f; }
      continue;
    }
    const int* fv = L.fv[order] + 3 * f;
    vertex_idx[3 * i] = __ldg(fv + 2);
    vertex_idx[3 * i + 1] = __ldg(fv + 1);
    vertex_idx[3 * i + 2] = __ldg(fv);
    if (nearest) {  // sphere.cpp:1107-1112: the strictly largest weight wins, ties go to the first
      int m = 0;
      if (s > t && s > u) m = 0;
      else if (t > s && t > u) m = 1;
      else if (u > s && u > t) m = 2;
      weights[3 * i] = m == 0 ? 1.f : 0.f;
      weights[3 * i + 1] = m == 1 ? 1.f : 0.f;
      weights[3 * i + 2] = m == 2 ? 1.f : 0.f;
    } else {
      weights[3 * i] = s;
      weights[3 * i + 1] = t;
      weights[3 * i + 2] = u;
    }
  }
}

}  // namespace mc

using namespace mc;

extern "C" int mc_sphere_locate(const float* samples, int64_t n, int32_t order,
                                const float* const* vertices, const int32_t* const* face_vertices,
                                const int32_t* const* face_adjacent, const int32_t* num_faces,
                                int32_t nearest, int64_t* face_idx, int64_t* vertex_idx,
                                float* weights, void* stream) {
  if (!samples || n < 0 || order < 0 || order >= SPHERE_MAX_LEVELS || !vertices || !face_vertices ||
      !face_adjacent || !num_faces || !face_idx || !vertex_idx || !weights)
    return MC_ERR_BAD_ARG;
  if (n == 0) return MC_OK;
  SphereLevels L = {};
  for (int l = 0; l <= order; ++l) {
    if (!vertices[l] || !face_vertices[l] || !face_adjacent[l] || num_faces[l] <= 0) return MC_ERR_BAD_ARG;
    L.v[l] = vertices[l];
    L.fv[l] = face_vertices[l];
    L.fadj[l] = face_adjacent[l];
    L.nf[l] = num_faces[l];
  }
  sphere_locate_kernel<<<grid_for(n, 128), 128, 0, (cudaStream_t)stream>>>(
      samples, (long)n, order, L, nearest, face_idx, vertex_idx, weights), MC_COUNT(1);
  MC_CHECK_LAUNCH();
  return MC_OK;
}
