/* oracle.c -- CPU restatement of the reference's hot-path arithmetic. TEST INFRASTRUCTURE ONLY.
 *
 * Nothing in the product may call into this file: it exists so that tests/, __graft_entry__.smoke() and bench.py's
 * cpu_baseline leg can check the CUDA kernels against an independent, plain-loop statement of the same maths.
 * Every function cites the reference file it follows. Accumulation is in double so the oracle is closer to the true
 * value than any float32 implementation; comparisons use max|err|/max|ref| <= 1e-4, the metric of the reference's own
 * checks (tools/gemm_bench.py:37, notes/scripts/conv_kinds_check.py:10).
 *
 * Parity pin: the reference's oracle is PyTorch's CPU aten (tools/acceptance.py:84-98, tools/gemm_bench.py:35-38). The
 * fixtures under tests/golden/ were produced by aten on the shape lists of the reference's check scripts and, for the
 * loss curves, by the reference's own model definitions; tests/test_oracle.py holds this file to them.
 * All tensors are float32, NCHW contiguous.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define IDX4(n, c, h, w, C, H, W) ((((int64_t)(n) * (C) + (c)) * (H) + (h)) * (W) + (w))

/* ---- dense convolution ------------------------------------------------------------------------------------------ */

/* y = conv(x, w) + bias, optional ReLU: kind 0 of omarchy_mac_torch/gemm.py:25-42 (aval/bval/store). */
void orc_conv_fwd(const float* x, const float* w, const float* bias, float* y, int n, int ci, int co, int ih, int iw, int ks,
                  int stride, int pad, int relu) {
  int oh = (ih + 2 * pad - ks) / stride + 1, ow = (iw + 2 * pad - ks) / stride + 1;
  for (int b = 0; b < n; b++)
    for (int o = 0; o < co; o++)
      for (int oy = 0; oy < oh; oy++)
        for (int ox = 0; ox < ow; ox++) {
          double s = bias ? bias[o] : 0.0;
          for (int c = 0; c < ci; c++)
            for (int ky = 0; ky < ks; ky++) {
              int yy = oy * stride + ky - pad;
              if (yy < 0 || yy >= ih) continue;
              for (int kx = 0; kx < ks; kx++) {
                int xx = ox * stride + kx - pad;
                if (xx < 0 || xx >= iw) continue;
                s += (double)x[IDX4(b, c, yy, xx, ci, ih, iw)] * w[IDX4(o, c, ky, kx, ci, ks, ks)];
              }
            }
          if (relu && s < 0) s = 0;
          y[IDX4(b, o, oy, ox, co, oh, ow)] = (float)s;
        }
}

/* dx by the definition: kind 1 of omarchy_mac_torch/gemm.py:43-59 (taps off the stride grid contribute nothing). */
void orc_conv_dgrad(const float* gy, const float* w, float* dx, int n, int ci, int co, int ih, int iw, int ks, int stride, int pad) {
  int oh = (ih + 2 * pad - ks) / stride + 1, ow = (iw + 2 * pad - ks) / stride + 1;
  for (int b = 0; b < n; b++)
    for (int c = 0; c < ci; c++)
      for (int y = 0; y < ih; y++)
        for (int x = 0; x < iw; x++) {
          double s = 0;
          for (int o = 0; o < co; o++)
            for (int ky = 0; ky < ks; ky++) {
              int yy = y + pad - ky;
              if (yy < 0 || yy % stride) continue;
              yy /= stride;
              if (yy >= oh) continue;
              for (int kx = 0; kx < ks; kx++) {
                int xx = x + pad - kx;
                if (xx < 0 || xx % stride) continue;
                xx /= stride;
                if (xx >= ow) continue;
                s += (double)gy[IDX4(b, o, yy, xx, co, oh, ow)] * w[IDX4(o, c, ky, kx, ci, ks, ks)];
              }
            }
          dx[IDX4(b, c, y, x, ci, ih, iw)] = (float)s;
        }
}

/* dx by stride phases: the host loop of csrc/conv.cpp:78-95 with the kind-5 loaders of omarchy_mac_torch/gemm.py:60-80.
 * Must equal orc_conv_dgrad exactly in index coverage; pins the phase algebra the CUDA kernels reuse. */
void orc_conv_dgrad_phases(const float* gy, const float* w, float* dx, int n, int ci, int co, int ih, int iw, int ks, int stride,
                           int pad) {
  int s = stride, oh = (ih + 2 * pad - ks) / s + 1, ow = (iw + 2 * pad - ks) / s + 1;
  for (int py = 0; py < s; py++)
    for (int px = 0; px < s; px++) {
      int hi = (ih - py + s - 1) / s, wi = (iw - px + s - 1) / s;
      if (hi <= 0 || wi <= 0) continue;
      int ky0 = (py + pad) % s, kx0 = (px + pad) % s;
      int jy = ky0 < ks ? (ks - ky0 + s - 1) / s : 0, jx = kx0 < ks ? (ks - kx0 + s - 1) / s : 0;
      int qy = (py + pad - ky0) / s, qx = (px + pad - kx0) / s;
      for (int b = 0; b < n; b++)
        for (int c = 0; c < ci; c++)
          for (int i = 0; i < hi; i++)
            for (int j = 0; j < wi; j++) {
              double acc = 0;
              for (int o = 0; o < co; o++)
                for (int ty = 0; ty < jy; ty++) {
                  int oy = i + qy - ty;
                  if (oy < 0 || oy >= oh) continue;
                  for (int tx = 0; tx < jx; tx++) {
                    int ox = j + qx - tx;
                    if (ox < 0 || ox >= ow) continue;
                    acc += (double)gy[IDX4(b, o, oy, ox, co, oh, ow)] * w[IDX4(o, c, ky0 + s * ty, kx0 + s * tx, ci, ks, ks)];
                  }
                }
              dx[IDX4(b, c, py + s * i, px + s * j, ci, ih, iw)] = (float)acc;
            }
    }
}

/* dw = sum over (n,oy,ox) gy * im2col(x): kind 2 of omarchy_mac_torch/gemm.py:81-91 + gemm_reduce.wgsl. */
void orc_conv_wgrad(const float* x, const float* gy, float* dw, int n, int ci, int co, int ih, int iw, int ks, int stride, int pad) {
  int oh = (ih + 2 * pad - ks) / stride + 1, ow = (iw + 2 * pad - ks) / stride + 1;
  for (int o = 0; o < co; o++)
    for (int c = 0; c < ci; c++)
      for (int ky = 0; ky < ks; ky++)
        for (int kx = 0; kx < ks; kx++) {
          double s = 0;
          for (int b = 0; b < n; b++)
            for (int oy = 0; oy < oh; oy++) {
              int yy = oy * stride + ky - pad;
              if (yy < 0 || yy >= ih) continue;
              for (int ox = 0; ox < ow; ox++) {
                int xx = ox * stride + kx - pad;
                if (xx < 0 || xx >= iw) continue;
                s += (double)gy[IDX4(b, o, oy, ox, co, oh, ow)] * x[IDX4(b, c, yy, xx, ci, ih, iw)];
              }
            }
          dw[IDX4(o, c, ky, kx, ci, ks, ks)] = (float)s;
        }
}

/* split-K slicing of the reference host (csrc/conv.cpp:106-109): returns slices, writes kslice. */
int orc_wgrad_slices(int64_t M, int64_t N, int64_t K, int bm, int bn, double mult, int64_t* kslice) {
  int64_t tiles = ((M + bm - 1) / bm) * ((N + bn - 1) / bn);
  int64_t want = (int64_t)(512 / tiles * mult), lim = K / 64;
  int64_t slices = want < lim ? want : lim;
  if (slices < 1) slices = 1;
  int64_t per = (K + slices - 1) / slices;
  *kslice = (per + 15) / 16 * 16;
  return (int)((K + *kslice - 1) / *kslice);
}

/* db[c] = sum gy: csrc/kernels/csum_nchw.wgsl. */
void orc_bias_grad(const float* gy, float* db, int n, int c, int hw) {
  for (int ch = 0; ch < c; ch++) {
    double s = 0;
    for (int b = 0; b < n; b++)
      for (int e = 0; e < hw; e++) s += gy[((int64_t)b * c + ch) * hw + e];
    db[ch] = (float)s;
  }
}

/* ---- depthwise: dwg_fwd.wgsl / dwg_gin.wgsl / dwg_gwt.wgsl (dw_*.wgsl are the stride-1 "same" case) ----------------- */

void orc_dw_fwd(const float* x, const float* w, const float* bias, float* y, int n, int c, int ih, int iw, int ks, int stride, int pad) {
  int oh = (ih + 2 * pad - ks) / stride + 1, ow = (iw + 2 * pad - ks) / stride + 1;
  for (int b = 0; b < n; b++)
    for (int ch = 0; ch < c; ch++)
      for (int oy = 0; oy < oh; oy++)
        for (int ox = 0; ox < ow; ox++) {
          double s = bias ? bias[ch] : 0.0;
          for (int ky = 0; ky < ks; ky++) {
            int sy = oy * stride - pad + ky;
            if (sy < 0 || sy >= ih) continue;
            for (int kx = 0; kx < ks; kx++) {
              int sx = ox * stride - pad + kx;
              if (sx < 0 || sx >= iw) continue;
              s += (double)x[IDX4(b, ch, sy, sx, c, ih, iw)] * w[((int64_t)ch * ks + ky) * ks + kx];
            }
          }
          y[IDX4(b, ch, oy, ox, c, oh, ow)] = (float)s;
        }
}
void orc_dw_dgrad(const float* gy, const float* w, float* dx, int n, int c, int ih, int iw, int ks, int stride, int pad) {
  int oh = (ih + 2 * pad - ks) / stride + 1, ow = (iw + 2 * pad - ks) / stride + 1;
  for (int b = 0; b < n; b++)
    for (int ch = 0; ch < c; ch++)
      for (int yy = 0; yy < ih; yy++)
        for (int xx = 0; xx < iw; xx++) {
          double s = 0;
          for (int ky = 0; ky < ks; ky++) {
            int ty = yy + pad - ky;
            if (ty < 0 || ty % stride || ty / stride >= oh) continue;
            for (int kx = 0; kx < ks; kx++) {
              int tx = xx + pad - kx;
              if (tx < 0 || tx % stride || tx / stride >= ow) continue;
              s += (double)gy[IDX4(b, ch, ty / stride, tx / stride, c, oh, ow)] * w[((int64_t)ch * ks + ky) * ks + kx];
            }
          }
          dx[IDX4(b, ch, yy, xx, c, ih, iw)] = (float)s;
        }
}
void orc_dw_wgrad(const float* x, const float* gy, float* dw, int n, int c, int ih, int iw, int ks, int stride, int pad) {
  int oh = (ih + 2 * pad - ks) / stride + 1, ow = (iw + 2 * pad - ks) / stride + 1;
  for (int ch = 0; ch < c; ch++)
    for (int ky = 0; ky < ks; ky++)
      for (int kx = 0; kx < ks; kx++) {
        double s = 0;
        for (int b = 0; b < n; b++)
          for (int oy = 0; oy < oh; oy++) {
            int yy = oy * stride + ky - pad;
            if (yy < 0 || yy >= ih) continue;
            for (int ox = 0; ox < ow; ox++) {
              int xx = ox * stride + kx - pad;
              if (xx < 0 || xx >= iw) continue;
              s += (double)gy[IDX4(b, ch, oy, ox, c, oh, ow)] * x[IDX4(b, ch, yy, xx, c, ih, iw)];
            }
          }
        dw[((int64_t)ch * ks + ky) * ks + kx] = (float)s;
      }
}

/* ---- batch norm ------------------------------------------------------------------------------------------------------- */

/* Shifted, split statistics exactly as the shaders do them, in float32 and in their summation structure:
 * bn_stats_part.wgsl:22-31 (S slices over the batch, shift = x[ch*hw]) then bn_stats_fin.wgsl:15-21 (mean, biased var,
 * running update with corr = count/(count-1) from csrc/nn.cpp:44). rm/rv may be NULL. */
void orc_bn_stats(const float* x, int n, int c, int hw, float momentum, float* mean, float* var, float* rm, float* rv) {
  int S = n >= 8 ? 8 : 1;
  double count = (double)n * hw;
  float corr = (float)(count / (count - 1 > 1 ? count - 1 : 1));
  for (int ch = 0; ch < c; ch++) {
    float shift = x[(int64_t)ch * hw];
    double s1 = 0, s2 = 0;
    for (int sl = 0; sl < S; sl++)
      for (int b = sl; b < n; b += S)
        for (int e = 0; e < hw; e++) {
          double d = (double)x[((int64_t)b * c + ch) * hw + e] - shift;
          s1 += d;
          s2 += d * d;
        }
    double a = s1 / count, m = shift + a, v = s2 / count - a * a;
    if (v < 0) v = 0;
    mean[ch] = (float)m;
    var[ch] = (float)v;
    if (rm) {
      rm[ch] = rm[ch] + momentum * ((float)m - rm[ch]);
      rv[ch] = rv[ch] + momentum * ((float)v * corr - rv[ch]);
    }
  }
}
/* y = (x-mean)*invstd*gamma+beta (+ReLU): bn_apply.wgsl:17-18, bn_relu.wgsl:17-18. */
void orc_bn_apply(const float* x, float* y, int n, int c, int hw, const float* mean, const float* invstd, const float* gamma,
                  const float* beta, int relu) {
  for (int b = 0; b < n; b++)
    for (int ch = 0; ch < c; ch++)
      for (int e = 0; e < hw; e++) {
        int64_t i = ((int64_t)b * c + ch) * hw + e;
        double r = ((double)x[i] - mean[ch]) * invstd[ch] * gamma[ch] + beta[ch];
        if (relu && r < 0) r = 0;
        y[i] = (float)r;
      }
}
/* Backward: bnb_reduce.wgsl:25-37 + bnb_apply.wgsl:19-21; with relu != 0 the gradient is first masked by y > 0 as in
 * bn_bwd_part.wgsl:25-38 and bn_bwd_apply.wgsl:19-23. dgb = [dgamma | dbeta]. dx may be NULL. */
void orc_bn_backward(const float* g, const float* x, const float* y, float* dx, int n, int c, int hw, const float* mean,
                     const float* invstd, const float* gamma, float* dgb, int relu) {
  double m = (double)n * hw;
  for (int ch = 0; ch < c; ch++) {
    double s1 = 0, s2 = 0;
    for (int b = 0; b < n; b++)
      for (int e = 0; e < hw; e++) {
        int64_t i = ((int64_t)b * c + ch) * hw + e;
        double gz = (relu && !(y[i] > 0.f)) ? 0.0 : g[i];
        s1 += gz;
        s2 += gz * ((double)x[i] - mean[ch]) * invstd[ch];
      }
    dgb[ch] = (float)s2;
    dgb[c + ch] = (float)s1;
    if (!dx) continue;
    for (int b = 0; b < n; b++)
      for (int e = 0; e < hw; e++) {
        int64_t i = ((int64_t)b * c + ch) * hw + e;
        double gz = (relu && !(y[i] > 0.f)) ? 0.0 : g[i];
        double xhat = ((double)x[i] - mean[ch]) * invstd[ch];
        dx[i] = (float)(gamma[ch] * invstd[ch] / m * (m * gz - s1 - xhat * s2));
      }
  }
}
/* Eval BN folded into conv weights: fold_bn, csrc/fused.cpp:34-40. cb may be NULL. */
void orc_fold_bn(const float* cw, const float* cb, const float* gamma, const float* beta, const float* rm, const float* rv, float eps,
                 int co, int per, float* fw, float* fb) {
  for (int o = 0; o < co; o++) {
    double scale = gamma[o] / sqrt((double)rv[o] + eps);
    for (int k = 0; k < per; k++) fw[(int64_t)o * per + k] = (float)(cw[(int64_t)o * per + k] * scale);
    fb[o] = (float)(((cb ? cb[o] : 0.0) - rm[o]) * scale + beta[o]);
  }
}

/* ---- pooling ------------------------------------------------------------------------------------------------------------ */

/* 2x2 stride-2 max pool with idx in {0..3}, strict > so the first maximum wins: pool_fwd.wgsl:15-21. */
void orc_pool2_fwd(const float* x, float* y, uint8_t* idx, int nc, int h, int w) {
  int oh = h / 2, ow = w / 2;
  for (int p = 0; p < nc; p++)
    for (int oy = 0; oy < oh; oy++)
      for (int ox = 0; ox < ow; ox++) {
        const float* b = x + ((int64_t)p * h + 2 * oy) * w + 2 * ox;
        float best = b[0];
        int bi = 0;
        if (b[1] > best) { best = b[1]; bi = 1; }
        if (b[w] > best) { best = b[w]; bi = 2; }
        if (b[w + 1] > best) { best = b[w + 1]; bi = 3; }
        y[((int64_t)p * oh + oy) * ow + ox] = best;
        idx[((int64_t)p * oh + oy) * ow + ox] = (uint8_t)bi;
      }
}
/* pool_bwd.wgsl:14-21 */
void orc_pool2_bwd(const float* g, const uint8_t* idx, float* gx, int nc, int h, int w) {
  int oh = h / 2, ow = w / 2;
  for (int p = 0; p < nc; p++)
    for (int yy = 0; yy < h; yy++)
      for (int xx = 0; xx < w; xx++) {
        int oy = yy / 2, ox = xx / 2;
        float v = 0;
        if (oy < oh && ox < ow) {
          int64_t o = ((int64_t)p * oh + oy) * ow + ox;
          if (idx[o] == (yy % 2) * 2 + xx % 2) v = g[o];
        }
        gx[((int64_t)p * h + yy) * w + xx] = v;
      }
}
/* General max pool, int64 flat index, NaN propagates: maxpool_gen_fwd.wgsl:16-28. */
void orc_maxpool_fwd(const float* x, float* y, int64_t* idx, int nc, int ih, int iw, int oh, int ow, int kh, int kw, int sh, int sw,
                     int ph, int pw, int dh, int dw) {
  for (int p = 0; p < nc; p++)
    for (int oy = 0; oy < oh; oy++)
      for (int ox = 0; ox < ow; ox++) {
        float best = -INFINITY;
        int64_t bi = -1;
        int stop = 0;
        for (int ky = 0; ky < kh && !stop; ky++) {
          int yy = oy * sh + ky * dh - ph;
          if (yy < 0 || yy >= ih) continue;
          for (int kx = 0; kx < kw; kx++) {
            int xx = ox * sw + kx * dw - pw;
            if (xx < 0 || xx >= iw) continue;
            float v = x[((int64_t)p * ih + yy) * iw + xx];
            if (bi < 0 || isnan(v) || v > best) {
              best = v;
              bi = (int64_t)yy * iw + xx;
              if (isnan(v)) { stop = 1; break; }
            }
          }
        }
        y[((int64_t)p * oh + oy) * ow + ox] = best;
        idx[((int64_t)p * oh + oy) * ow + ox] = bi;
      }
}
/* maxpool_gen_bwd.wgsl (scatter form: identical result) */
void orc_maxpool_bwd(const float* g, const int64_t* idx, float* gx, int nc, int ih, int iw, int oh, int ow) {
  memset(gx, 0, sizeof(float) * (size_t)nc * ih * iw);
  for (int p = 0; p < nc; p++)
    for (int o = 0; o < oh * ow; o++) {
      int64_t k = idx[(int64_t)p * oh * ow + o];
      if (k >= 0) gx[(int64_t)p * ih * iw + k] += g[(int64_t)p * oh * ow + o];
    }
}
/* adaptive average pool: adapool_fwd.wgsl (window [floor(o*I/O), ceil((o+1)*I/O))). */
void orc_adapool_fwd(const float* x, float* y, int nc, int ih, int iw, int oh, int ow) {
  for (int p = 0; p < nc; p++)
    for (int oy = 0; oy < oh; oy++)
      for (int ox = 0; ox < ow; ox++) {
        int y0 = (oy * ih) / oh, y1 = ((oy + 1) * ih + oh - 1) / oh, x0 = (ox * iw) / ow, x1 = ((ox + 1) * iw + ow - 1) / ow;
        double s = 0;
        for (int yy = y0; yy < y1; yy++)
          for (int xx = x0; xx < x1; xx++) s += x[((int64_t)p * ih + yy) * iw + xx];
        y[((int64_t)p * oh + oy) * ow + ox] = (float)(s / ((y1 - y0) * (x1 - x0)));
      }
}

/* ---- optimizers ----------------------------------------------------------------------------------------------------------- */

/* sgd.wgsl:9-24, float32 arithmetic as the shader does it. m may be NULL when momentum == 0. */
void orc_sgd(float* p, const float* g, float* m, int64_t numel, float lr, float mom, float damp, float wd, int nesterov, int first,
             int maximize) {
  for (int64_t i = 0; i < numel; i++) {
    float gr = g[i];
    if (maximize) gr = -gr;
    float pv = p[i];
    gr = gr + wd * pv;
    float d = gr;
    if (mom != 0.f) {
      float v = gr;
      if (!first) v = mom * m[i] + (1.f - damp) * gr;
      m[i] = v;
      d = nesterov ? gr + mom * v : v;
    }
    p[i] = pv - lr * d;
  }
}
/* adam.wgsl:13-27; `step` is the already incremented step count. */
void orc_adam(float* p, const float* g, float* m, float* v, int64_t numel, float step, float lr, float b1, float b2, float eps,
              float wd, int decoupled, int maximize) {
  float bc1 = 1.f - powf(b1, step), sbc2 = sqrtf(1.f - powf(b2, step));
  for (int64_t i = 0; i < numel; i++) {
    float gr = g[i];
    if (maximize) gr = -gr;
    float pv = p[i];
    if (decoupled) pv = pv * (1.f - lr * wd); else gr = gr + wd * pv;
    float mi = m[i] + (1.f - b1) * (gr - m[i]);
    float vi = b2 * v[i] + (1.f - b2) * gr * gr;
    m[i] = mi;
    v[i] = vi;
    p[i] = pv - (lr / bc1) * mi / (sqrtf(vi) / sbc2 + eps);
  }
}
