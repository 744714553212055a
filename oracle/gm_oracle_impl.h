/* Body of the CPU oracle, included once per floating type (T, SUFFIX).
 * TEST INFRASTRUCTURE ONLY -- see gm_oracle.c. */

/* Descriptor rows (n, a_n per head, flat offset, coefficient offset, dim):
 * reference src/gm_attention/nn/fused/attention.h:57-63. */

/* Raw score of edge e for head h: sum over frequencies and the head's copies of
 * <q_i, tau_n k_j> (attention.h:145-165), descriptor rows ascending, copies ascending. */
static T FN(score)(const T* q_i, const T* k_j, const T* tau, const int64_t* desc, int F, int h) {
  T acc = 0;
  for (int f = 0; f < F; ++f) {
    const int n = (int)desc[5 * f], a_n = (int)desc[5 * f + 1], off = (int)desc[5 * f + 2];
    if (n == 0) {
      const int base = off + h * a_n;
      for (int c = 0; c < a_n; ++c) acc += q_i[base + c] * k_j[base + c];
    } else {
      const T tr = tau[2 * n], ti = tau[2 * n + 1];
      const int base = off + 2 * h * a_n;
      for (int c = 0; c < a_n; ++c) {
        const T kr = k_j[base + 2 * c], ki = k_j[base + 2 * c + 1];
        acc += q_i[base + 2 * c] * (tr * kr - ti * ki) + q_i[base + 2 * c + 1] * (tr * ki + ti * kr);
      }
    }
  }
  return acc;
}

/* alpha (E, H): attention.h:295-316.  Masked edges (inside = 0) are left out
 * of both the shift and the sum and get alpha = 0. */
void FN(oracle_softmax_forward)(const T* q, const T* k, const T* transport, const T* bias, const uint8_t* inside,
                                const int64_t* desc, const int64_t* row_ptr, const int64_t* source, int64_t n_nodes, int D,
                                int F, int orders, int H, T scale, T* alpha) {
  for (int64_t i = 0; i < n_nodes; ++i) {
    const int64_t e0 = row_ptr[i], e1 = row_ptr[i + 1];
    for (int h = 0; h < H; ++h) {
      T m = -INFINITY;
      for (int64_t e = e0; e < e1; ++e) {
        const T lw = scale * FN(score)(q + i * D, k + source[e] * D, transport + e * orders * 2, desc, F, h) + bias[e];
        alpha[e * H + h] = lw;
        if (inside[e] && lw > m) m = lw;
      }
      T sum = 0;
      for (int64_t e = e0; e < e1; ++e) {
        const T u = inside[e] ? EXP(alpha[e * H + h] - m) : 0;
        alpha[e * H + h] = u;
        sum += u;
      }
      for (int64_t e = e0; e < e1; ++e) alpha[e * H + h] /= sum;
    }
  }
}

/* Which descriptor row / head / partner a flat column belongs to (attention.h:111-130). */
static int FN(locate)(const int64_t* desc, int F, int H, int c, int* n, int* h, int* part, int* a, int* a_n, int* coff) {
  for (int f = 0; f < F; ++f) {
    const int mult = (int)desc[5 * f + 1], off = (int)desc[5 * f + 2], dim = (int)desc[5 * f + 4];
    if (c >= off && c < off + H * mult * dim) {
      const int local = c - off, copy = local / dim;
      *n = (int)desc[5 * f]; *h = copy / mult; *a = copy % mult; *part = local % dim; *a_n = mult; *coff = (int)desc[5 * f + 3];
      return 1;
    }
  }
  return 0;
}

/* dq (written), dk (accumulated into a zeroed buffer): attention.h:320-348. */
void FN(oracle_softmax_backward)(const T* dalpha, const T* q, const T* k, const T* transport, const int64_t* desc,
                                 const int64_t* row_ptr, const int64_t* source, const T* alpha, int64_t n_nodes, int D, int F,
                                 int orders, int H, T scale, T* dq, T* dk) {
  for (int64_t x = 0; x < n_nodes * D; ++x) dk[x] = 0;
  for (int64_t i = 0; i < n_nodes; ++i) {
    const int64_t e0 = row_ptr[i], e1 = row_ptr[i + 1];
    T total[8] = {0};
    for (int h = 0; h < H; ++h)
      for (int64_t e = e0; e < e1; ++e) total[h] += alpha[e * H + h] * dalpha[e * H + h];
    for (int c = 0; c < D; ++c) {
      int n, h, part, a, a_n, coff;
      T acc = 0;
      if (FN(locate)(desc, F, H, c, &n, &h, &part, &a, &a_n, &coff)) {
        for (int64_t e = e0; e < e1; ++e) {
          const int64_t j = source[e];
          const T ds = scale * alpha[e * H + h] * (dalpha[e * H + h] - total[h]);
          if (n == 0) {
            acc += ds * k[j * D + c];
            dk[j * D + c] += ds * q[i * D + c];
          } else {
            const T tr = transport[(e * orders + n) * 2], ti = transport[(e * orders + n) * 2 + 1];
            const int re = c - part;
            const T kr = k[j * D + re], ki = k[j * D + re + 1], qr = q[i * D + re], qi = q[i * D + re + 1];
            acc += ds * (part == 0 ? tr * kr - ti * ki : tr * ki + ti * kr);          /* tau k */
            dk[j * D + c] += ds * (part == 0 ? tr * qr + ti * qi : tr * qi - ti * qr); /* conj(tau) q */
          }
        }
      }
      dq[i * D + c] = acc;
    }
  }
}

static T FN(rho_power)(T rho, int n) { /* (r/c)^{2n} by repeated multiplication: attention.h:137-142 */
  T s = 1;
  for (int x = 0; x < 2 * n; ++x) s *= rho;
  return s;
}

/* Depthwise convolution under given weights: message attention.h:174-206, node walk :265-275. */
void FN(oracle_conv_forward)(const T* v, const T* rc, const T* cc, const T* transport, const T* angular, const T* rho,
                             const T* weights, const int64_t* desc, const int64_t* row_ptr, const int64_t* source,
                             int64_t n_nodes, int D, int F, int orders, int A0, int W, T* out) {
  for (int64_t i = 0; i < n_nodes; ++i)
    for (int c = 0; c < D; ++c) {
      int n, h, part, a, a_n, coff;
      T y = 0;
      if (FN(locate)(desc, F, 1, c, &n, &h, &part, &a, &a_n, &coff)) {
        for (int64_t e = row_ptr[i]; e < row_ptr[i + 1]; ++e) {
          const int64_t j = source[e];
          T msg;
          if (n == 0) {
            msg = rc[e * A0 + a] * v[j * D + c];
          } else {
            const T tr = transport[(e * orders + n) * 2], ti = transport[(e * orders + n) * 2 + 1];
            const T vr = v[j * D + c - part], vi = v[j * D + c - part + 1];
            const T zr = tr * vr - ti * vi, zi = tr * vi + ti * vr;
            const T* co = cc + e * W + coff;
            const T Ar = co[2 * a], Ai = co[2 * a + 1], Br = co[2 * a_n + 2 * a], Bi = co[2 * a_n + 2 * a + 1];
            const T p = FN(rho_power)(rho[e], n);
            const T wr = p * angular[(e * orders + 2 * n) * 2], wi = p * angular[(e * orders + 2 * n) * 2 + 1];
            const T bzr = Br * zr + Bi * zi, bzi = Bi * zr - Br * zi; /* B conj(z) */
            const T mr = (Ar * zr - Ai * zi) + (wr * bzr - wi * bzi), mi = (Ar * zi + Ai * zr) + (wr * bzi + wi * bzr);
            msg = part == 0 ? mr : mi;
          }
          y += weights[e] * msg;
        }
      }
      out[i * D + c] = y;
    }
}

/* Backward of the depthwise convolution: attention.h:211-232, :277-287. */
void FN(oracle_conv_backward)(const T* g, const T* v, const T* rc, const T* cc, const T* transport, const T* angular,
                              const T* rho, const T* weights, const int64_t* desc, const int64_t* row_ptr,
                              const int64_t* source, int64_t n_nodes, int D, int F, int orders, int A0, int W, T* dv, T* drc,
                              T* dcc) {
  for (int64_t x = 0; x < n_nodes * D; ++x) dv[x] = 0;
  for (int64_t i = 0; i < n_nodes; ++i)
    for (int c = 0; c < D; ++c) {
      int n, h, part, a, a_n, coff;
      if (!FN(locate)(desc, F, 1, c, &n, &h, &part, &a, &a_n, &coff)) continue;
      for (int64_t e = row_ptr[i]; e < row_ptr[i + 1]; ++e) {
        const int64_t j = source[e];
        if (n == 0) {
          const T dm = weights[e] * g[i * D + c];
          drc[e * A0 + a] = dm * v[j * D + c];
          dv[j * D + c] += dm * rc[e * A0 + a];
          continue;
        }
        const int re = c - part;
        const T tr = transport[(e * orders + n) * 2], ti = transport[(e * orders + n) * 2 + 1];
        const T vr = v[j * D + re], vi = v[j * D + re + 1];
        const T zr = tr * vr - ti * vi, zi = tr * vi + ti * vr;
        const int64_t ci = e * W + coff + 2 * a;
        const T Ar = cc[ci], Ai = cc[ci + 1], Br = cc[ci + 2 * a_n], Bi = cc[ci + 2 * a_n + 1];
        const T p = FN(rho_power)(rho[e], n);
        const T wr = p * angular[(e * orders + 2 * n) * 2], wi = p * angular[(e * orders + 2 * n) * 2 + 1];
        const T dmr = weights[e] * g[i * D + re], dmi = weights[e] * g[i * D + re + 1];
        const T dAr = dmr * zr + dmi * zi, dAi = dmi * zr - dmr * zi;     /* dm conj(z) */
        const T xr = dmr * wr + dmi * wi, xi = dmi * wr - dmr * wi;       /* dm conj(w) */
        const T dBr = xr * zr - xi * zi, dBi = xr * zi + xi * zr;
        dcc[ci + part] = part == 0 ? dAr : dAi;
        dcc[ci + 2 * a_n + part] = part == 0 ? dBr : dBi;
        const T bdr = Br * dmr + Bi * dmi, bdi = Bi * dmr - Br * dmi;     /* B conj(dm) */
        const T dzr = (Ar * dmr + Ai * dmi) + (wr * bdr - wi * bdi), dzi = (Ar * dmi - Ai * dmr) + (wr * bdi + wi * bdr);
        dv[j * D + c] += part == 0 ? tr * dzr + ti * dzi : tr * dzi - ti * dzr; /* conj(tau) dz */
      }
    }
}

/* The value path given alpha (E, H): out_i = sum_e alpha_e,h(c) * (tau_n(e) v_j)[c] -- the
 * reference's eager "gather, transport_field (nn/kernels.py:156-189), weight,
 * scatter_add_to_nodes (nn/_scatter.py:36-46)" for one sample. */
void FN(oracle_value_forward)(const T* alpha, const T* v, const T* transport, const int64_t* desc, const int64_t* row_ptr,
                              const int64_t* source, int64_t n_nodes, int D, int F, int orders, int H, T* out) {
  for (int64_t i = 0; i < n_nodes; ++i)
    for (int c = 0; c < D; ++c) {
      int n, h, part, a, a_n, coff;
      T y = 0;
      if (FN(locate)(desc, F, H, c, &n, &h, &part, &a, &a_n, &coff)) {
        for (int64_t e = row_ptr[i]; e < row_ptr[i + 1]; ++e) {
          const int64_t j = source[e];
          if (n == 0) {
            y += alpha[e * H + h] * v[j * D + c];
          } else {
            const T tr = transport[(e * orders + n) * 2], ti = transport[(e * orders + n) * 2 + 1];
            const T vr = v[j * D + c - part], vi = v[j * D + c - part + 1];
            y += alpha[e * H + h] * (part == 0 ? tr * vr - ti * vi : tr * vi + ti * vr);
          }
        }
      }
      out[i * D + c] = y;
    }
}

/* Its adjoint: dalpha_e,h = <dO_i, tau v_j>_h (zeroed here, then summed), dv_j += alpha conj(tau) dO_i (zeroed here). */
void FN(oracle_value_backward)(const T* dout, const T* alpha, const T* v, const T* transport, const int64_t* desc,
                               const int64_t* row_ptr, const int64_t* source, int64_t n_nodes, int D, int F, int orders, int H,
                               T* dalpha, T* dv) {
  const int64_t n_edges = row_ptr[n_nodes];
  for (int64_t x = 0; x < n_nodes * D; ++x) dv[x] = 0;
  for (int64_t x = 0; x < n_edges * H; ++x) dalpha[x] = 0;
  for (int64_t i = 0; i < n_nodes; ++i)
    for (int c = 0; c < D; ++c) {
      int n, h, part, a, a_n, coff;
      if (!FN(locate)(desc, F, H, c, &n, &h, &part, &a, &a_n, &coff)) continue;
      const T g = dout[i * D + c];
      for (int64_t e = row_ptr[i]; e < row_ptr[i + 1]; ++e) {
        const int64_t j = source[e];
        if (n == 0) {
          dalpha[e * H + h] += g * v[j * D + c];
          dv[j * D + c] += alpha[e * H + h] * g;
        } else {
          const T tr = transport[(e * orders + n) * 2], ti = transport[(e * orders + n) * 2 + 1];
          const int re = c - part;
          const T vr = v[j * D + re], vi = v[j * D + re + 1];
          dalpha[e * H + h] += g * (part == 0 ? tr * vr - ti * vi : tr * vi + ti * vr);
          /* d/dv of g * (tau v)[c]: the real part picks (tr, -ti) on (vr, vi), the imaginary part (ti, tr) */
          if (part == 0) { dv[j * D + re] += alpha[e * H + h] * g * tr; dv[j * D + re + 1] -= alpha[e * H + h] * g * ti; }
          else           { dv[j * D + re] += alpha[e * H + h] * g * ti; dv[j * D + re + 1] += alpha[e * H + h] * g * tr; }
        }
      }
    }
}

/* The fused layer = oracle_softmax_forward then oracle_value_forward, per sample.  `alpha` is caller
 * scratch (E, H).  The geometry describes one sample; `batch` samples of n_nodes rows share it. */
void FN(oracle_attention_forward)(const T* q, const T* k, const T* v, const T* transport, const T* bias,
                                  const uint8_t* inside, const int64_t* desc, const int64_t* row_ptr, const int64_t* source,
                                  int64_t n_nodes, int64_t batch, int D, int F, int orders, int H, T scale, T* alpha, T* out) {
  for (int64_t b = 0; b < batch; ++b) {
    const int64_t o = b * n_nodes * D;
    FN(oracle_softmax_forward)(q + o, k + o, transport, bias, inside, desc, row_ptr, source, n_nodes, D, F, orders, H, scale, alpha);
    FN(oracle_value_forward)(alpha, v + o, transport, desc, row_ptr, source, n_nodes, D, F, orders, H, out + o);
  }
}

/* Backward of the fused layer by the chain rule through the two stages.  alpha, dalpha: caller scratch (E, H). */
void FN(oracle_attention_backward)(const T* dout, const T* q, const T* k, const T* v, const T* transport, const T* bias,
                                   const uint8_t* inside, const int64_t* desc, const int64_t* row_ptr, const int64_t* source,
                                   int64_t n_nodes, int64_t batch, int D, int F, int orders, int H, T scale, T* alpha,
                                   T* dalpha, T* dq, T* dk, T* dv) {
  for (int64_t b = 0; b < batch; ++b) {
    const int64_t o = b * n_nodes * D;
    FN(oracle_softmax_forward)(q + o, k + o, transport, bias, inside, desc, row_ptr, source, n_nodes, D, F, orders, H, scale, alpha);
    FN(oracle_value_backward)(dout + o, alpha, v + o, transport, desc, row_ptr, source, n_nodes, D, F, orders, H, dalpha, dv + o);
    FN(oracle_softmax_backward)(dalpha, q + o, k + o, transport, desc, row_ptr, source, alpha, n_nodes, D, F, orders, H, scale,
                                dq + o, dk + o);
  }
}
