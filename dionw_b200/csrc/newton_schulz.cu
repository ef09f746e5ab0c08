// The Newton-Schulz product schedules, launched product by product on the
// tcgen05 GEMMs of gemm.cu.
#include "common.cuh"

namespace dionw {

int symmetric_product(const void* a, const void* b, int64_t blocks, int64_t m, int64_t kdim, int64_t lda,
                      int64_t a_batch, int64_t ldb, int64_t b_batch, const void* cin, int64_t ldc, int64_t cin_batch, float alpha, float beta, void* out,
                      int64_t ldo, int64_t out_batch, void* out2, float diag, int dtype, cudaStream_t stream);
int batched_gemm(const void* a, int64_t lda, int64_t a_batch, const void* b, int64_t ldb, int64_t b_batch,
                 bool b_is_nk, const void* cin, int64_t ldc, int64_t cin_batch, float beta, void* out, int64_t ldo,
                 int64_t out_batch, int64_t blocks, int64_t m, int64_t n, int64_t kdim, int in_dtype, int out_dtype,
                 float* rowsq, cudaStream_t stream);

namespace {

struct Coeff {
  double a, b, c;
};

// Polar Express coefficients divided by the safety factor 1.05, 1.05^3, 1.05^5:
// the table the reference's Gram iteration uses.
constexpr double kS = 1.05;
const Coeff kGram[5] = {
    {8.28721201814563 / kS, -23.595886519098837 / (kS * kS * kS), 17.300387312530933 / (kS * kS * kS * kS * kS)},
    {4.107059111542203 / kS, -2.9478499167379106 / (kS * kS * kS), 0.5448431082926601 / (kS * kS * kS * kS * kS)},
    {3.9486908534822946 / kS, -2.908902115962949 / (kS * kS * kS), 0.5518191394370137 / (kS * kS * kS * kS * kS)},
    {3.3184196573706015 / kS, -2.488488024314874 / (kS * kS * kS), 0.51004894012372 / (kS * kS * kS * kS * kS)},
    {2.300652019954817 / kS, -1.6689039845747493 / (kS * kS * kS), 0.4188073119525673 / (kS * kS * kS * kS * kS)},
};
const Coeff kPolarExpress[5] = {
    {8.156554524902461, -22.48329292557795, 15.878769915207462},
    {4.042929935166739, -2.808917465908714, 0.5000178451051316},
    {3.8916678022926607, -2.772484153217685, 0.5060648178503393},
    {3.285753657755655, -2.3681294933425376, 0.46449024233003106},
    {2.3465413258596377, -1.7097828382687081, 0.42323551169305323},
};
const Coeff kKeller[5] = {
    {3.4445, -4.7750, 2.0315}, {3.4445, -4.7750, 2.0315}, {3.4445, -4.7750, 2.0315},
    {3.4445, -4.7750, 2.0315}, {3.4445, -4.7750, 2.0315},
};
constexpr int kRestart = 2;

inline int64_t round_up(int64_t v, int64_t to) { return (v + to - 1) / to * to; }
inline size_t align256(size_t v) { return (v + 255) / 256 * 256; }

struct Layout {
  int64_t ldg;          // leading dimension of the m x m scratch matrices
  size_t x_bytes;       // one [blocks, m, ldx] operand
  size_t g_bytes;       // one [blocks, m, ldg] matrix
  bool wide_gram;
};

Layout layout_of(int64_t blocks, int64_t m, int64_t n, int64_t ldx, int kind) {
  Layout l;
  l.ldg = round_up(m, 8);
  l.x_bytes = align256(size_t(blocks) * m * ldx * 2);
  l.g_bytes = align256(size_t(blocks) * m * l.ldg * 2);
  l.wide_gram = (kind == DIONW_NS_GRAM || kind == DIONW_NS_GRAM_FULL) && n > m;
  return l;
}

size_t bytes_of(const Layout& l) {
  // Gram on wide blocks: X1 + {G, Z, Q0, Q1, RZ}.  Standard iteration: X1, X2 + {G, P}.
  return l.wide_gram ? l.x_bytes + 5 * l.g_bytes : 2 * l.x_bytes + 2 * l.g_bytes;
}


}  // namespace
}  // namespace dionw

extern "C" size_t dionw_newton_schulz_workspace_bytes(int64_t blocks, int64_t m, int64_t n, int kind) {
  using namespace dionw;
  if (blocks <= 0 || m <= 0 || n <= 0) return 0;
  return bytes_of(layout_of(blocks, m, n, round_up(n, 8), kind)) + 256;
}

extern "C" int64_t dionw_newton_schulz_rowsq_parts(int64_t n) { return n <= 0 ? 0 : 2 * ((n + 255) / 256); }

extern "C" int dionw_newton_schulz(void* x, void* out, int64_t blocks, int64_t m, int64_t n, int64_t ldx, int kind,
                                   void* workspace, size_t workspace_bytes, float* rowsq, void* stream_ptr) {
  using namespace dionw;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  DIONW_REQUIRE(kind == DIONW_NS_GRAM || kind == DIONW_NS_POLAR_EXPRESS || kind == DIONW_NS_KELLER ||
                    kind == DIONW_NS_GRAM_FULL,
                "newton_schulz: unknown kind %d", kind);
  DIONW_REQUIRE(blocks > 0 && m > 0 && n >= m, "newton_schulz: needs blocks > 0 and 0 < m <= n (got %lld, %lld, %lld)",
                (long long)blocks, (long long)m, (long long)n);
  DIONW_REQUIRE(ldx >= n && ldx % 8 == 0, "newton_schulz: ldx must be >= n and a multiple of 8");
  DIONW_REQUIRE(aligned16(x) && aligned16(out), "newton_schulz: x and out must be 16-byte aligned");
  const Layout l = layout_of(blocks, m, n, ldx, kind);
  uint8_t* ws = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(workspace) + 255) & ~uintptr_t(255));
  const size_t lost = size_t(ws - reinterpret_cast<uint8_t*>(workspace));
  if (workspace == nullptr || workspace_bytes < bytes_of(l) + lost) {
    set_error("newton_schulz: workspace of %zu bytes is smaller than the %zu needed", workspace_bytes,
              bytes_of(l) + lost);
    return DIONW_ERR_WORKSPACE;
  }
  const bool gram = kind == DIONW_NS_GRAM || kind == DIONW_NS_GRAM_FULL;
  const int dt = gram ? DIONW_F16 : DIONW_BF16;
  // Every m x m matrix of the Gram schedule is a polynomial in one symmetric G, so the
  // products among them are symmetric too: GRAM computes their lower tiles and mirrors,
  // GRAM_FULL computes them as general products, as the reference's cuBLAS calls do.
  const bool mirror = kind == DIONW_NS_GRAM;
  const int64_t xb = m * ldx;       // batch strides in elements
  const int64_t gb = m * l.ldg;
  const int64_t ldg = l.ldg;
  int st = DIONW_OK;
#define DIONW_STEP(call)            \
  do {                              \
    st = (call);                    \
    if (st != DIONW_OK) return st;  \
  } while (0)

  if (l.wide_gram) {
    void* x0 = x;
    void* x1 = ws;
    void* g = ws + l.x_bytes;
    void* z = ws + l.x_bytes + l.g_bytes;
    void* q0 = ws + l.x_bytes + 2 * l.g_bytes;
    void* q1 = ws + l.x_bytes + 3 * l.g_bytes;
    void* rz = ws + l.x_bytes + 4 * l.g_bytes;
    void* xcur = x0;
    void* q = q0;
    void* qnext = q1;
    // G = X X^T
    DIONW_STEP(symmetric_product(xcur, nullptr, blocks, m, n, ldx, xb, 0, 0, nullptr, 0, 0, 1.0f, 0.0f, g, ldg, gb, nullptr, 0.0f,
                                 dt, stream));
    for (int i = 0; i < 5; ++i) {
      const Coeff k = kGram[i];
      if (i == kRestart) {
        // X <- Q X, G <- X X^T
        DIONW_STEP(batched_gemm(q, ldg, gb, xcur, ldx, xb, false, nullptr, 0, 0, 0.0f, x1, ldx, xb, blocks, m, n, m,
                                dt, dt, nullptr, stream));
        xcur = x1;
        DIONW_STEP(symmetric_product(xcur, nullptr, blocks, m, n, ldx, xb, 0, 0, nullptr, 0, 0, 1.0f, 0.0f, g, ldg, gb,
                                     nullptr, 0.0f, dt, stream));
      }
      const bool fresh_q = (i == 0 || i == kRestart);
      // Z = c G G^T + b G; on a fresh start also Q = Z + a I.  The diagonal is round(fp32(Z) + fp32(a)),
      // as the reference's compiled GPU step forms `z + a * eye` (its eager CPU run rounds `a` to
      // fp16 first, which costs 4e-3 of accuracy on 256 x 4096 operands).
      DIONW_STEP(symmetric_product(g, nullptr, blocks, m, m, ldg, gb, 0, 0, g, ldg, gb, float(k.c), float(k.b), z, ldg, gb,
                                   fresh_q ? q : nullptr, float(k.a), dt, stream));
      if (!fresh_q) {
        // Q <- a Q + Q Z   (Z is stored symmetric, so Z^T == Z bit for bit)
        if (mirror)
          DIONW_STEP(symmetric_product(q, z, blocks, m, m, ldg, gb, ldg, gb, q, ldg, gb, 1.0f, float(k.a), qnext, ldg,
                                       gb, nullptr, 0.0f, dt, stream));
        else
          DIONW_STEP(batched_gemm(q, ldg, gb, z, ldg, gb, true, q, ldg, gb, float(k.a), qnext, ldg, gb, blocks, m,
                                  m, m, dt, dt, nullptr, stream));
        void* t = q;
        q = qnext;
        qnext = t;
      }
      if (i < 4 && i + 1 != kRestart) {
        // RZ = a G + G Z ; G <- a RZ + Z RZ
        if (mirror) {
          DIONW_STEP(symmetric_product(g, z, blocks, m, m, ldg, gb, ldg, gb, g, ldg, gb, 1.0f, float(k.a), rz, ldg,
                                       gb, nullptr, 0.0f, dt, stream));
          DIONW_STEP(symmetric_product(z, rz, blocks, m, m, ldg, gb, ldg, gb, rz, ldg, gb, 1.0f, float(k.a), g, ldg,
                                       gb, nullptr, 0.0f, dt, stream));
        } else {
          DIONW_STEP(batched_gemm(g, ldg, gb, z, ldg, gb, true, g, ldg, gb, float(k.a), rz, ldg, gb, blocks, m, m,
                                  m, dt, dt, nullptr, stream));
          DIONW_STEP(batched_gemm(z, ldg, gb, rz, ldg, gb, false, rz, ldg, gb, float(k.a), g, ldg, gb, blocks, m,
                                  m, m, dt, dt, nullptr, stream));
        }
      }
    }
    // out = Q X in bf16
    DIONW_STEP(batched_gemm(q, ldg, gb, xcur, ldx, xb, false, nullptr, 0, 0, 0.0f, out, ldx, xb, blocks, m, n, m, dt,
                            DIONW_BF16, rowsq, stream));
    return DIONW_OK;
  }

  // Standard iteration: X <- a X + (b G + c G^2) X with G = X X^T.
  const Coeff* table = gram ? kGram : (kind == DIONW_NS_POLAR_EXPRESS ? kPolarExpress : kKeller);
  void* x1 = ws;
  void* x2 = ws + l.x_bytes;
  void* g = ws + 2 * l.x_bytes;
  void* poly = ws + 2 * l.x_bytes + l.g_bytes;
  void* cur = x;
  for (int i = 0; i < 5; ++i) {
    const Coeff k = table[i];
    void* next = (i == 4) ? out : ((cur == x1) ? x2 : x1);
    DIONW_STEP(symmetric_product(cur, nullptr, blocks, m, n, ldx, xb, 0, 0, nullptr, 0, 0, 1.0f, 0.0f, g, ldg, gb, nullptr, 0.0f,
                                 dt, stream));
    DIONW_STEP(symmetric_product(g, nullptr, blocks, m, m, ldg, gb, 0, 0, g, ldg, gb, float(k.c), float(k.b), poly, ldg, gb,
                                 nullptr, 0.0f, dt, stream));
    DIONW_STEP(batched_gemm(poly, ldg, gb, cur, ldx, xb, false, cur, ldx, xb, float(k.a), next, ldx, xb, blocks, m,
                            n, m, dt, i == 4 ? DIONW_BF16 : dt, i == 4 ? rowsq : nullptr, stream));
    cur = next;
  }
#undef DIONW_STEP
  return DIONW_OK;
}
