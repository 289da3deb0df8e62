// Lane-cooperative complex FFT: a line of N = R*Q points shared by Q neighbouring lane groups of
// a warp, used by the N = 64 / 128 single-call 2-D transforms (fft2d_coop.cu) and the N = 256
// two-pass forward transform (fft2d_256.cu).
#pragma once
#include "fft_regs.cuh"

namespace fbfft_b200 {

// Length-N = R*Q complex FFT shared by Q lanes (lane index bits above log2(32/Q)
// select q; Q = 1 is a plain in-register FFT).  In: a[m*P + jl] = x[jl + P*q + R*m],
// P = R/Q.  Out: a[brev(k, R)] = X[Q*k + q].  lf[qq] = exp(-+2*pi*i*q*qq/(Q*Q)) is
// the part of the twiddle that depends on the lane.
template <int N, int R, int Q, bool INV, bool PK = INV>
__device__ __forceinline__ void coop_fft(float2 (&a)[R], int q, const float2 (&lf)[Q]) {
  if constexpr (Q == 1) {
    fft_bitrev<R, INV, PK>(a);
  } else {
    constexpr int P = R / Q;
    constexpr int LP = 32 / Q;  // lanes per q group
    constexpr int LOGQ = ilog2c(Q);
    // radix-Q step over m for every jl: output qq lands at a[brev(qq, Q)*P + jl]
    static_for<P>([&](auto jc) {
      constexpr int jl = decltype(jc)::value;
      Dif<Q, jl, P, INV, R, PK>::run(a);
    });
    float2 c[R];
    static_for<Q>([&](auto qc) {
      constexpr int qq = decltype(qc)::value;
      static_for<P>([&](auto jc) {
        constexpr int jl = decltype(jc)::value;
        float2 v = mul_tw<jl * qq, N, INV>(a[brev(qq, Q) * P + jl]);
        if (qq > 0) v = cmul(v, lf[qq]);
        c[qq * P + jl] = v;
      });
    });
    // all-to-all between the Q lanes: block qq goes to lane qq; afterwards block i holds
    // what lane i sent, i.e. c[i*P + jl] is element j = jl + P*i of this lane's R-point input
    static_for<LOGQ>([&](auto tc) {
      constexpr int t = decltype(tc)::value;
      const bool mybit = (q >> t) & 1;
      static_for<Q / 2>([&](auto ic) {
        constexpr int idx = decltype(ic)::value;
        constexpr int i0 = ((idx >> t) << (t + 1)) | (idx & ((1 << t) - 1));
        constexpr int i1 = i0 | (1 << t);
        static_for<P>([&](auto jc) {
          constexpr int jl = decltype(jc)::value;
          const float2 lo = c[i0 * P + jl], hi = c[i1 * P + jl];
          const float sx = mybit ? lo.x : hi.x, sy = mybit ? lo.y : hi.y;
          const float rx = __shfl_xor_sync(0xffffffffu, sx, LP << t);
          const float ry = __shfl_xor_sync(0xffffffffu, sy, LP << t);
          c[i0 * P + jl] = mybit ? make_float2(rx, ry) : lo;
          c[i1 * P + jl] = mybit ? hi : make_float2(rx, ry);
        });
      });
    });
    fft_bitrev<R, INV, PK>(c);
#pragma unroll
    for (int i = 0; i < R; ++i) a[i] = c[i];
  }
}

template <int Q, bool INV>
__device__ __forceinline__ void lane_factors(int q, float2 (&lf)[Q]) {
#pragma unroll
  for (int qq = 0; qq < Q; ++qq) {
    float s, c;
    sincospif((INV ? 2.0f : -2.0f) * (float)(q * qq) / (float)(Q * Q), &s, &c);
    lf[qq] = make_float2(c, s);
  }
}

}  // namespace fbfft_b200
