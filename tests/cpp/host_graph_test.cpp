// Operator-level tests of the C++ host mirror, written the way the reference tests its operators
// (src/tests/units/operator_tests.cpp:508-534 "dot product", :618-659 "affine transformation"): build an
// expression graph from hand-made parameters, forward(), read the values back.  Here B is an intgemm8
// parameter, the product runs on the GPU engine, and the expected values come from the CPU checker
// (oracle/oracle_i8.c), compared bit for bit.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <vector>

#include <cuda_runtime.h>

#include "../../include/marian_i8.h"
#include "../../marian-dev_b200/host/marian_graph.h"

extern "C" {
float mo_prepare_b(const float* w, int k, int n, int w_is_nk, int8_t* bt);
int mo_affine(const float* a, int m, int k, const int8_t* bt, float qb, int n, const float* bias, float scale, int relu, float* out,
              int8_t* aq_out, int32_t* acc_out, float* qa_out);
size_t mo_p8_packed_bytes(int K, int N);
int mo_p8_prepare_b(const float* w, int K, int N, int8_t* packed);
int mo_p8_gemm_packed(const float* a, const int8_t* packed, const float* bias, float* c, int M, int N, int K);
}

using namespace marian;

static int failures = 0;
#define CHECK(cond)                                                       \
  do {                                                                    \
    if(!(cond)) {                                                         \
      std::printf("CHECK failed: %s (line %d)\n", #cond, __LINE__);       \
      ++failures;                                                         \
    }                                                                     \
  } while(0)

template <typename F>
static bool aborts_with(F f, const char* needle) {
  try {
    f();
  } catch(const MarianRuntimeException& e) {
    return std::string(e.what()).find(needle) != std::string::npos;
  }
  return false;
}

int main() {
  void *arena = nullptr, *ws = nullptr;
  const size_t arenaBytes = size_t(256) << 20, wsBytes = mi8_workspace_bytes(0, 0, 0);
  if(cudaMalloc(&arena, arenaBytes) != cudaSuccess || cudaMalloc(&ws, wsBytes) != cudaSuccess) {
    std::printf("no CUDA device memory\n");
    return 2;
  }

  {  // "affine transformation": A [4,3] . B [3,2] + bias [1,2], small integers as in the reference's test; K padded to 16
     // with zeros (the int8 kernels need K % 16 == 0, intgemm itself needs K % 64 == 0)
    ExpressionGraph graph(arena, arenaBytes, ws, wsBytes);
    std::vector<float> vA(4 * 16, 0.f), vB(16 * 2, 0.f), vBias = {2, 3};
    const float a3[12] = {1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12}, b3[6] = {1, 2, 3, 4, 5, 6};
    for(int i = 0; i < 4; ++i)
      for(int j = 0; j < 3; ++j)
        vA[i * 16 + j] = a3[i * 3 + j] * (127.f / 12.f);   // max|A| -> 127
    for(int i = 0; i < 3; ++i)
      for(int j = 0; j < 2; ++j)
        vB[i * 2 + j] = b3[i * 2 + j] * (127.f / 6.f);
    Expr A = graph.param("A", {4, 16}, Type::float32, vA.data());
    Expr Bf = graph.param("B", {16, 2}, Type::float32, vB.data());
    Expr bias = graph.param("bias", {1, 2}, Type::float32, vBias.data());
    Expr B = graph.intgemm8Param("B_intgemm8", Bf);
    CHECK(B->shape() == Shape({16, 2}) && B->value_type() == Type::intgemm8);
    Expr C = affine(A, B, bias);
    Expr D = dot(A, B, false, false, 0.5f);
    Expr R = affineWithReluDropout(A, B, bias);
    CHECK(C->shape() == Shape({4, 2}));
    graph.forward();
    std::vector<float> vC, vD, vR;
    graph.get(C, vC);
    graph.get(D, vD);
    graph.get(R, vR);
    const float expect[8] = {22, 28, 49, 64, 76, 100, 103, 136};  // A3 . B3
    const float s = (127.f / 12.f) * (127.f / 6.f);
    const float tol = 0.02f * 136.f * s;  // int8 precision: each operand is rounded to 1/127 of its maximum
    for(int i = 0; i < 8; ++i) {
      CHECK(std::fabs(vC[i] - (expect[i] * s + vBias[i % 2])) <= tol);
      CHECK(std::fabs(vD[i] - 0.5f * expect[i] * s) <= tol);
      CHECK(vR[i] == (vC[i] > 0 ? vC[i] : 0.f));
    }
  }

  {  // random operands, [2,5,64] x [64,40]: bit-exact against the CPU checker, output keeps the leading dimensions
    ExpressionGraph graph(arena, arenaBytes, ws, wsBytes);
    std::mt19937 rng(7);
    std::normal_distribution<float> nd(0.f, 1.f);
    const int M = 10, K = 64, N = 40;
    std::vector<float> vA(M * K), vB(K * N), vBias(N);
    for(auto& v : vA) v = nd(rng);
    for(auto& v : vB) v = 0.02f * nd(rng);
    for(auto& v : vBias) v = 0.01f * nd(rng);
    Expr A = graph.param("x", {2, 5, K}, Type::float32, vA.data());
    Expr W = graph.intgemm8Param("ffn_W1", graph.param("ffn_W1_f", {K, N}, Type::float32, vB.data()));
    Expr b = graph.param("ffn_b1", {1, N}, Type::float32, vBias.data());
    Expr Y = affineWithReluDropout(A, W, b);
    CHECK(Y->shape() == Shape({2, 5, N}));
    graph.forward();
    std::vector<float> got;
    graph.get(Y, got);
    std::vector<int8_t> bt(N * K);
    const float qb = mo_prepare_b(vB.data(), K, N, 0, bt.data());
    std::vector<float> want(M * N);
    mo_affine(vA.data(), M, K, bt.data(), qb, N, vBias.data(), 1.f, 1, want.data(), nullptr, nullptr, nullptr);
    bool same = true;
    for(int i = 0; i < M * N; ++i)
      same = same && got[i] == want[i];
    CHECK(same);
    std::vector<int8_t> gotBt;
    float gotQb = 0;
    graph.get(W, gotBt, &gotQb);
    CHECK(gotQb == qb && gotBt == bt);
  }

  {  // transA: A arrives as [K, M] and is transposed by a node of its own before the quantisation, as the reference does
     // (intgemm_interface.h:52); values equal the product with the pre-transposed operand, bit for bit
    ExpressionGraph graph(arena, arenaBytes, ws, wsBytes);
    std::mt19937 rng(11);
    std::normal_distribution<float> nd(0.f, 1.f);
    const int M = 37, K = 48, N = 24;
    std::vector<float> vA(M * K), vAt(K * M), vB(K * N), vBias(N);
    for(auto& v : vA) v = nd(rng);
    for(int i = 0; i < M; ++i)
      for(int j = 0; j < K; ++j)
        vAt[j * M + i] = vA[i * K + j];
    for(auto& v : vB) v = 0.02f * nd(rng);
    for(auto& v : vBias) v = 0.01f * nd(rng);
    Expr At = graph.param("At", {K, M}, Type::float32, vAt.data());
    Expr W = graph.intgemm8Param("W", graph.param("W_f", {K, N}, Type::float32, vB.data()));
    Expr b = graph.param("b", {1, N}, Type::float32, vBias.data());
    Expr Y = affine(At, W, b, /*transA=*/true);
    Expr D = dot(At, W, true, false, 2.f);
    CHECK(Y->shape() == Shape({M, N}) && D->shape() == Shape({M, N}));
    graph.forward();
    std::vector<float> got, gotD;
    graph.get(Y, got);
    graph.get(D, gotD);
    std::vector<int8_t> bt(N * K);
    const float qb = mo_prepare_b(vB.data(), K, N, 0, bt.data());
    std::vector<float> want(M * N), wantD(M * N);
    mo_affine(vA.data(), M, K, bt.data(), qb, N, vBias.data(), 1.f, 0, want.data(), nullptr, nullptr, nullptr);
    mo_affine(vA.data(), M, K, bt.data(), qb, N, nullptr, 2.f, 0, wantD.data(), nullptr, nullptr, nullptr);
    bool same = true;
    for(int i = 0; i < M * N; ++i)
      same = same && got[i] == want[i] && gotD[i] == wantD[i];
    CHECK(same);
  }

  {  // packed8avx512 weights: converted in the graph and uploaded as a ready item; affine and dot dispatch on isPacked(B)
    ExpressionGraph graph(arena, arenaBytes, ws, wsBytes);
    const int M = 10, K = 512, N = 96;
    std::mt19937 rng(9);
    std::normal_distribution<float> nd(0.f, 1.f);
    std::vector<float> vA(M * K), vB(K * N), vBias(N);
    for(auto& v : vA) v = nd(rng) * 2.f;
    for(auto& v : vB) v = nd(rng) * 0.05f;
    for(auto& v : vBias) v = nd(rng) * 0.1f;
    std::vector<int8_t> item(mo_p8_packed_bytes(K, N));
    CHECK(mo_p8_prepare_b(vB.data(), K, N, item.data()) == 0);
    std::vector<float> want(M * N), wantDot(M * N);
    mo_p8_gemm_packed(vA.data(), item.data(), vBias.data(), want.data(), M, N, K);
    mo_p8_gemm_packed(vA.data(), item.data(), nullptr, wantDot.data(), M, N, K);
    Expr A = graph.param("A", {2, 5, K}, Type::float32, vA.data());
    Expr Bf = graph.param("encoder_l1_ffn_W1", {K, N}, Type::float32, vB.data());
    Expr bias = graph.param("encoder_l1_ffn_b1", {1, N}, Type::float32, vBias.data());
    Expr W = graph.packed8Param("encoder_l1_ffn_W1", Bf);                       // converted on the device
    Expr W2 = graph.packed8Item("encoder_l1_ffn_W1", {K, N}, item.data());      // as read from a model file
    CHECK(W->value_type() == Type::packed8avx512 && isPacked(W->value_type()) && W->shape() == Shape({K, N}));
    Expr Y = affine(A, W, bias), Y2 = affine(A, W2, bias), D = dot(A, W2);
    CHECK(Y->shape() == Shape({2, 5, N}));
    graph.forward();
    std::vector<float> got, got2, gotDot;
    graph.get(Y, got);
    graph.get(Y2, got2);
    graph.get(D, gotDot);
    bool same = true;
    for(int i = 0; i < M * N; ++i)
      same = same && got[i] == want[i] && got2[i] == want[i] && gotDot[i] == wantDot[i];
    CHECK(same);
    CHECK(aborts_with([&] { affine(A, W, bias, false, true); }, "Transposition is currently not supported"));
    CHECK(aborts_with([&] { gpu::variant::affine(Type::packed8avx2, A, W, W->shape(), bias, false, false, 1.f); }, "Only avx512 packed matrix format"));
    std::vector<float> v8(4 * 256, 1.f);
    Expr A8 = graph.param("A8", {4, 256}, Type::float32, v8.data());
    CHECK(aborts_with([&] { affine(A8, W, nullptr); }, "Inner dimensions"));
  }

  {  // error behaviour: the reference's messages for wrongly typed operands
    ExpressionGraph graph(arena, arenaBytes, ws, wsBytes);
    std::vector<float> v(16 * 16, 1.f);
    Expr A = graph.param("A", {16, 16}, Type::float32, v.data());
    Expr Bf = graph.param("B", {16, 16}, Type::float32, v.data());
    Expr B = graph.intgemm8Param("B_q", Bf);
    CHECK(aborts_with([&] { affine(A, Bf, nullptr); }, "GPU only supports float"));
    CHECK(aborts_with([&] { gpu::integer::affineOrDot(B, B, nullptr, false, false, 1.f); }, "Intgemm expects type of A to be float32 not intgemm8"));
    CHECK(aborts_with([&] { gpu::integer::affineOrDot(A, A, nullptr, false, false, 1.f); }, "Intgemm expects type of B to be a variant of intgemm not float32"));
    CHECK(aborts_with([&] { affineWithReluDropout(A, B, nullptr, 0.1f); }, "inference-only"));
    std::vector<float> v8(16 * 8, 1.f);
    Expr A8 = graph.param("A8", {16, 8}, Type::float32, v8.data());
    CHECK(aborts_with([&] { affine(A8, B, nullptr); }, "Inner dimensions"));
  }

  cudaFree(arena);
  cudaFree(ws);
  if(failures == 0)
    std::printf("host graph tests passed\n");
  return failures == 0 ? 0 : 1;
}
