// Python extension module "GNNAdvisor": the reference's operator API
// (EPPGCN/GCNConv/EPPGCN.cpp:388-403) on top of the eppgcn_b200 C-ABI.
//
// Every function keeps the reference's name, positional arguments and return
// shape.  Differences, all towards exactness or safety:
//   * work is enqueued on torch's current stream and the per-epoch operators do
//     not block the host (the reference synchronises after every kernel);
//   * CUDA failures raise RuntimeError instead of calling exit();
//   * build_part returns int32 tensors (the reference returns float32, exact
//     only below 2^24; callers apply .int() either way) and always closes the
//     last group (EPPGCN.cpp:222-223 skips that when the last vertex is empty);
//   * compact_back_edge reports valid_len in a float64 tensor (float32 in the
//     reference, EPPGCN.cpp:293-294);
//   * split_back_part is exact for any degree (the reference handles at most
//     1023 parts per vertex, cuCompactor.cu:500,527) and returns num_edges + 1
//     entries, one more than the reference, so the closing pointer always fits.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <cstdlib>
#include <mutex>
#include <vector>

#include "eppgcn_b200.h"

namespace {

#define CHECK_CUDA(x) TORCH_CHECK(x.is_cuda(), #x " must be a CUDA tensor")
#define CHECK_CONTIGUOUS(x) TORCH_CHECK(x.is_contiguous(), #x " must be contiguous")
#define CHECK_INPUT(x) CHECK_CUDA(x); CHECK_CONTIGUOUS(x)
#define CHECK_I32(x) TORCH_CHECK(x.scalar_type() == at::kInt, #x " must be an int32 tensor")
#define CHECK_F32(x) TORCH_CHECK(x.scalar_type() == at::kFloat, #x " must be a float32 tensor")
#define CHECK_BOOL(x) TORCH_CHECK(x.scalar_type() == at::kBool, #x " must be a bool tensor")

void epp_check(int status, const char *what) {
  TORCH_CHECK(status == EPP_OK, what, " failed: ", eppgcn_status_string(status), ": ", eppgcn_last_error());
}

void *current_stream() { return static_cast<void *>(at::cuda::getCurrentCUDAStream().stream()); }

// RAII pair of timer marks on the current stream.
struct ScopedTime {
  int slot, category, layer;
  ScopedTime(int category_, int layer_ = 0) : slot(eppgcn_time_begin(current_stream())), category(category_), layer(layer_) {}
  ~ScopedTime() { eppgcn_time_end(slot, category, layer, current_stream()); }
};

int padded_width(int64_t dim) { return static_cast<int>((dim + 7) / 8 * 8); }

// ---------------------------------------------------------------------------
// Aggregation plans.  The operators receive the same edge lists epoch after
// epoch (the CSR for `forward`, the compacted path of a layer for
// `ours_backward`), so the tile plan of an edge list is prepared at its first
// use and found again by the identity of the tensors that describe it: data
// pointers, sizes and in-place modification counters.  A handful of plans is
// kept (a model has one forward list and one backward list per layer); the
// least recently used one goes when there are more.
// EPPGCN_B200_GROUP_KERNEL=1 in the environment turns the plans off: every
// aggregation then runs the stateless group kernel.
// ---------------------------------------------------------------------------
struct PlanKey {
  const void *a, *b;
  int64_t na, nb, rows, edges;
  uint32_t va, vb;
  int device;
  bool operator==(const PlanKey &o) const {
    return a == o.a && b == o.b && na == o.na && nb == o.nb && rows == o.rows && edges == o.edges && va == o.va &&
           vb == o.vb && device == o.device;
  }
};

struct PlanEntry {
  PlanKey key;
  eppgcn_tile_plan *plan;
  torch::Tensor buffer;      // the plan's device arrays
  torch::Tensor keep_a, keep_b;   // the key's tensors: while they live here their addresses cannot be handed out again
  uint64_t last_use;
};

class PlanCache {
 public:
  static constexpr size_t kCapacity = 16;

  // Finds the plan of `key`, or builds it with `build(buffer_ptr, buffer_bytes, &plan)`.
  template <typename Build>
  const eppgcn_tile_plan *get(const PlanKey &key, const torch::Tensor &key_a, const torch::Tensor &key_b,
                              int64_t edges, int64_t rows, int64_t sources, Build build) {
    const auto opts = key_a.options();
    std::lock_guard<std::mutex> lock(mu_);
    for (PlanEntry &e : entries_)
      if (e.key == key) {
        e.last_use = ++clock_;
        return e.plan;
      }
    const size_t bytes = eppgcn_tile_plan_bytes(edges, static_cast<int>(rows), static_cast<int>(sources));
    auto buffer = at::empty({static_cast<int64_t>((bytes + 7) / 8)}, opts.dtype(at::kLong));
    eppgcn_tile_plan *plan = nullptr;
    epp_check(build(buffer.data_ptr(), bytes, &plan), "eppgcn_tile_plan");
    if (entries_.size() >= kCapacity) {
      size_t oldest = 0;
      for (size_t i = 1; i < entries_.size(); ++i)
        if (entries_[i].last_use < entries_[oldest].last_use) oldest = i;
      eppgcn_tile_plan_destroy(entries_[oldest].plan);
      entries_.erase(entries_.begin() + static_cast<std::ptrdiff_t>(oldest));
    }
    entries_.push_back(PlanEntry{key, plan, buffer, key_a, key_b, ++clock_});
    return plan;
  }

  void clear() {
    std::lock_guard<std::mutex> lock(mu_);
    for (PlanEntry &e : entries_) eppgcn_tile_plan_destroy(e.plan);
    entries_.clear();
  }

  size_t size() {
    std::lock_guard<std::mutex> lock(mu_);
    return entries_.size();
  }

 private:
  std::mutex mu_;
  std::vector<PlanEntry> entries_;
  uint64_t clock_ = 0;
};

// Never destroyed: its tensors must not be released after the CUDA context has gone at exit.
PlanCache &plan_cache() {
  static PlanCache *cache = new PlanCache();
  return *cache;
}

bool plans_enabled() {
  const char *v = std::getenv("EPPGCN_B200_GROUP_KERNEL");
  return !(v && v[0] && v[0] != '0');
}

const eppgcn_tile_plan *forward_plan(const torch::Tensor &row_pointers, const torch::Tensor &column_index) {
  const int64_t n = row_pointers.numel() - 1, e = column_index.numel();
  PlanKey key{row_pointers.data_ptr(), column_index.data_ptr(), row_pointers.numel(), column_index.numel(), n, e,
              static_cast<uint32_t>(row_pointers._version()), static_cast<uint32_t>(column_index._version()),
              row_pointers.get_device()};
  return plan_cache().get(key, row_pointers, column_index, e, n, n, [&](void *buf, size_t bytes, eppgcn_tile_plan **plan) {
    return eppgcn_tile_plan_from_csr(plan, buf, bytes, row_pointers.data_ptr<int>(), column_index.data_ptr<int>(),
                                     static_cast<int>(n), e, static_cast<int>(n), current_stream());
  });
}

const eppgcn_tile_plan *backward_plan(const torch::Tensor &id, const torch::Tensor &partPointer,
                                      const torch::Tensor &edgeList, int numParts, int64_t n) {
  // the path's edge count closes the part pointers; it is read once, when the plan is made
  PlanKey key{id.data_ptr(), edgeList.data_ptr(), id.numel(), partPointer.numel(), n, numParts,
              static_cast<uint32_t>(id._version()), static_cast<uint32_t>(edgeList._version()), id.get_device()};
  return plan_cache().get(key, id, edgeList, id.numel(), n, n, [&](void *buf, size_t bytes, eppgcn_tile_plan **plan) {
    const int64_t valid = numParts > 0 ? partPointer[numParts].item<int>() : 0;
    TORCH_CHECK(valid >= 0 && valid <= id.numel() && valid <= edgeList.numel(),
                "partPointer[numParts] is not an edge count of the compacted lists");
    return eppgcn_tile_plan_from_ids(plan, buf, bytes, id.data_ptr<int>(), edgeList.data_ptr<int>(), valid,
                                     static_cast<int>(n), static_cast<int>(n), current_stream());
  });
}

// sum over the plan's edges of rows that already carry their source factor; destination factor `degrees`
torch::Tensor aggregate_planned(const eppgcn_tile_plan *plan, const torch::Tensor &src, const torch::Tensor &degrees,
                                int64_t n) {
  const int64_t d = src.size(1);
  auto out = at::empty({n, d}, src.options());
  if (n == 0) return out;
  epp_check(eppgcn_spmm_tiles(out.data_ptr<float>(), 0, src.data_ptr<float>(), src.stride(0), plan,
                              degrees.data_ptr<float>(), static_cast<int>(d), current_stream()),
            "eppgcn_spmm_tiles");
  return out;
}

// degrees[r] * x[r] for the rows the plan's edges name, in rows padded to 32 bytes
torch::Tensor pack_scaled(const eppgcn_tile_plan *plan, const torch::Tensor &x, const torch::Tensor &degrees) {
  const int64_t n = x.size(0), d = x.size(1), ld = padded_width(d);
  auto full = at::empty({n, ld}, x.options());
  if (n > 0)
    epp_check(eppgcn_pack_scaled_rows(full.data_ptr<float>(), ld, x.data_ptr<float>(), x.stride(0),
                                      degrees.data_ptr<float>(), plan, static_cast<int>(n), static_cast<int>(d),
                                      current_stream()),
              "eppgcn_pack_scaled_rows");
  return full.narrow(1, 0, d);
}

// diag(degrees) * (X @ W), written into rows whose stride is a multiple of 32
// bytes, so every gathered row starts on a sector boundary and can be fetched
// with 16-byte loads whatever the output width (22 classes -> 24 floats).  The
// source-side factor of the edge weight is folded in here, which saves the
// aggregation one gathered sector per edge.  Narrow outputs run the library's
// FP32 FMA kernel; anything else goes through cuBLAS and one scaling pass.
torch::Tensor update_scaled_padded(const torch::Tensor &x, const torch::Tensor &w, const torch::Tensor &degrees) {
  const int64_t n = x.size(0), k = x.size(1), d = w.size(1);
  const int64_t ld = padded_width(d);
  auto full = at::empty({n, ld}, x.options());
  auto view = full.narrow(1, 0, d);
  const bool aligned = x.stride(0) % 4 == 0 && reinterpret_cast<uintptr_t>(x.data_ptr<float>()) % 16 == 0;
  if (aligned && n > 0 && n < (1LL << 31)) {
    // 32 output columns per launch; the last block also clears the padding columns
    for (int64_t c0 = 0; c0 < d; c0 += 32) {
      const int cols = static_cast<int>(std::min<int64_t>(32, d - c0));
      const bool last = c0 + cols == d;
      epp_check(eppgcn_update_scaled(full.data_ptr<float>() + c0, ld, x.data_ptr<float>(), x.stride(0),
                                     w.data_ptr<float>() + c0, d, degrees.data_ptr<float>(), static_cast<int>(n),
                                     static_cast<int>(k), cols, last ? static_cast<int>(ld - d) : 0,
                                     current_stream()),
                "eppgcn_update_scaled");
    }
  } else {
    at::mm_out(view, x, w);
    view.mul_(degrees.narrow(0, 0, n).unsqueeze(1));
  }
  return view;
}

// The two dense products of a layer's backward (EPPGCN_kernel.cu:614-615):
//   d_input = d' @ W^T   [N, Din]      d_weight = X^T @ d'   [Din, Dout]
// Both are tall and skinny; the library's FP32 FMA kernels read X and write
// d_input once, where cuBLAS takes several times longer on these shapes.  Shapes
// outside the kernels' limits go through torch::mm.
std::vector<torch::Tensor> backward_update(const torch::Tensor &d_prime, const torch::Tensor &X,
                                           const torch::Tensor &W, const eppgcn_tile_plan *plan = nullptr,
                                           bool need_d_input = true) {
  const int64_t n = d_prime.size(0), dout = d_prime.size(1), din = W.size(0);
  const bool ok = n > 0 && n < (1LL << 31) && din % 4 == 0 && dout % 4 == 0 && X.stride(0) % 4 == 0 &&
                  reinterpret_cast<uintptr_t>(X.data_ptr<float>()) % 16 == 0 &&
                  reinterpret_cast<uintptr_t>(d_prime.data_ptr<float>()) % 16 == 0;
  const bool narrow_ok = n > 0 && n < (1LL << 31) && dout <= 32 && din * ((dout + 3) / 4 * 4) <= 4096 &&
                         din % 4 == 0 && X.stride(0) % 4 == 0 &&
                         reinterpret_cast<uintptr_t>(X.data_ptr<float>()) % 16 == 0 &&
                         reinterpret_cast<uintptr_t>(d_prime.data_ptr<float>()) % 16 == 0;
  if (!ok && !narrow_ok)
    return {need_d_input ? at::mm(d_prime, W.transpose(0, 1)) : at::empty({0}, d_prime.options()),
            at::mm(X.transpose(0, 1), d_prime)};
  torch::Tensor d_input = at::empty({0}, d_prime.options());
  if (need_d_input) {
    auto wt = W.transpose(0, 1).contiguous();                 // [Dout, Din]
    d_input = at::empty({n, din}, d_prime.options());
    for (int64_t c0 = 0; c0 < din; c0 += 32) {                // 32 output columns per launch
      const int cols = static_cast<int>(std::min<int64_t>(32, din - c0));
      epp_check(eppgcn_update_scaled(d_input.data_ptr<float>() + c0, din, d_prime.data_ptr<float>(), dout,
                                     wt.data_ptr<float>() + c0, din, nullptr, static_cast<int>(n),
                                     static_cast<int>(dout), cols, 0, current_stream()),
                "eppgcn_update_scaled");
    }
  }
  // d_weight: only the rows of the execution path face a non-zero row of d' (EPPGCN_kernel.cu:607,616
  // sketches the same restriction); wide shapes go block by block (32 columns of d', <= 128 of X)
  const int *rows = nullptr;
  int listed = 0;
  if (plan) epp_check(eppgcn_tile_plan_active_rows(plan, &rows, &listed), "eppgcn_tile_plan_active_rows");
  const bool by_rows = plan && listed < n;
  auto d_weight = at::empty({din, dout}, d_prime.options());
  const int64_t cb = std::min<int64_t>(dout, 32);
  const int64_t kb = std::max<int64_t>(4, std::min<int64_t>(din, 4096 / ((cb + 3) / 4 * 4) / 4 * 4));
  const bool whole = cb == dout && kb == din;
  for (int64_t c0 = 0; c0 < dout; c0 += cb) {
    const int cols = static_cast<int>(std::min<int64_t>(cb, dout - c0));
    for (int64_t k0 = 0; k0 < din; k0 += kb) {
      const int ks = static_cast<int>(std::min<int64_t>(kb, din - k0));
      auto block = whole ? d_weight : at::empty({ks, cols}, d_prime.options());
      const float *xp = X.data_ptr<float>() + k0, *dp = d_prime.data_ptr<float>() + c0;
      if (by_rows)
        epp_check(eppgcn_weight_grad_rows(block.data_ptr<float>(), xp, X.stride(0), dp, dout, rows, listed, ks, cols,
                                          current_stream()),
                  "eppgcn_weight_grad_rows");
      else
        epp_check(eppgcn_weight_grad(block.data_ptr<float>(), xp, X.stride(0), dp, dout, static_cast<int>(n), ks,
                                     cols, current_stream()),
                  "eppgcn_weight_grad");
      if (!whole) d_weight.narrow(0, k0, ks).narrow(1, c0, cols).copy_(block);
    }
  }
  return {d_input, d_weight};
}

torch::Tensor aggregate_forward(const torch::Tensor &feat, const torch::Tensor &row_pointers,
                                const torch::Tensor &column_index, const torch::Tensor &degrees,
                                const torch::Tensor &part_pointers, const torch::Tensor &part2Node,
                                int partSize, int dimWorker, int warpPerBlock, bool prescaled = false) {
  const int64_t n = feat.size(0), d = feat.size(1);
  TORCH_CHECK(row_pointers.numel() == n + 1, "row_pointers must have num_nodes + 1 entries");
  TORCH_CHECK(degrees.numel() >= n, "degrees must have one entry per vertex");
  TORCH_CHECK(part_pointers.numel() == part2Node.numel() + 1 || part2Node.numel() == 0,
              "part_pointers must have one more entry than part2Node");
  auto out = at::empty({n, d}, feat.options());
  const int64_t ld = n > 1 ? feat.stride(0) : std::max<int64_t>(feat.stride(0), d);
  epp_check(eppgcn_spmm_forward(out.data_ptr<float>(), 0, feat.data_ptr<float>(), ld,
                                row_pointers.data_ptr<int>(), column_index.data_ptr<int>(),
                                degrees.data_ptr<float>(), prescaled ? nullptr : degrees.data_ptr<float>(),
                                part_pointers.data_ptr<int>(), part2Node.data_ptr<int>(),
                                static_cast<int>(n), static_cast<int>(d), static_cast<int>(part2Node.numel()),
                                partSize, dimWorker, warpPerBlock, current_stream()),
            "eppgcn_spmm_forward");
  return out;
}

// forward(input, weight, row_pointers, column_index, degrees, part_pointers,
//         part2Node, partSize, dimWorker, warpPerBlock) -> [output]
// EPPGCN.cpp:79-102, EPPGCN_kernel.cu:123-202.
std::vector<torch::Tensor> spmm_forward(torch::Tensor input, torch::Tensor weight, torch::Tensor row_pointers,
                                        torch::Tensor column_index, torch::Tensor degrees,
                                        torch::Tensor part_pointers, torch::Tensor part2Node, int partSize,
                                        int dimWorker, int warpPerBlock) {
  CHECK_INPUT(input); CHECK_INPUT(weight); CHECK_INPUT(row_pointers); CHECK_INPUT(column_index);
  CHECK_INPUT(degrees); CHECK_INPUT(part_pointers); CHECK_INPUT(part2Node);
  CHECK_F32(input); CHECK_F32(weight); CHECK_F32(degrees);
  CHECK_I32(row_pointers); CHECK_I32(column_index); CHECK_I32(part_pointers); CHECK_I32(part2Node);
  c10::cuda::CUDAGuard guard(input.device());
  torch::Tensor tmp;
  {
    ScopedTime t(1);
    tmp = update_scaled_padded(input, weight, degrees);
  }
  ScopedTime t(0);
  if (plans_enabled() && input.size(0) > 0 && row_pointers.numel() == input.size(0) + 1)
    return {aggregate_planned(forward_plan(row_pointers, column_index), tmp, degrees, input.size(0))};
  return {aggregate_forward(tmp, row_pointers, column_index, degrees, part_pointers, part2Node, partSize,
                            dimWorker, warpPerBlock, /*prescaled=*/true)};
}

// backward(d_output, X, W, row_pointers, column_index, degrees, part_pointers,
//          part2Node, partSize, dimWorker, warpPerBlock) -> [d_input, d_weight]
// The uncompacted backward of EPPGCN.cpp:104-130, EPPGCN_kernel.cu:395-469.
std::vector<torch::Tensor> spmm_backward(torch::Tensor d_output, torch::Tensor X, torch::Tensor W,
                                         torch::Tensor row_pointers, torch::Tensor column_index,
                                         torch::Tensor degrees, torch::Tensor part_pointers,
                                         torch::Tensor part2Node, int partSize, int dimWorker,
                                         int warpPerBlock) {
  CHECK_INPUT(d_output); CHECK_INPUT(X); CHECK_INPUT(W); CHECK_INPUT(row_pointers); CHECK_INPUT(column_index);
  CHECK_INPUT(degrees); CHECK_INPUT(part_pointers); CHECK_INPUT(part2Node);
  CHECK_F32(d_output); CHECK_F32(X); CHECK_F32(W); CHECK_F32(degrees);
  CHECK_I32(row_pointers); CHECK_I32(column_index); CHECK_I32(part_pointers); CHECK_I32(part2Node);
  c10::cuda::CUDAGuard guard(d_output.device());
  torch::Tensor d_input_prime;
  {
    ScopedTime t(2, 0);
    if (plans_enabled() && d_output.size(0) > 0 && row_pointers.numel() == d_output.size(0) + 1) {
      const eppgcn_tile_plan *plan = forward_plan(row_pointers, column_index);
      d_input_prime = aggregate_planned(plan, pack_scaled(plan, d_output, degrees), degrees, d_output.size(0));
    } else {
      d_input_prime = aggregate_forward(d_output, row_pointers, column_index, degrees, part_pointers, part2Node,
                                        partSize, dimWorker, warpPerBlock);
    }
  }
  ScopedTime t(3);
  return backward_update(d_input_prime, X, W);
}

// mask_forward(id, partPointer, edgeList, src_mask, ngh_mask, backEdgeMask,
//              node_degs, num_layers, layer, blockx, blocky) -> None
// EPPGCN.cpp:132-155, EPPGCN_kernel.cu:297-388.
void mask_forward(torch::Tensor id, torch::Tensor partPointer, torch::Tensor edgeList, torch::Tensor src_mask,
                  torch::Tensor ngh_mask, torch::Tensor backEdgeMask, torch::Tensor node_degs, int num_layers,
                  int layer, int blockx, int blocky) {
  CHECK_INPUT(id); CHECK_INPUT(partPointer); CHECK_INPUT(edgeList); CHECK_INPUT(src_mask);
  CHECK_INPUT(ngh_mask); CHECK_INPUT(backEdgeMask); CHECK_INPUT(node_degs);
  CHECK_I32(id); CHECK_I32(partPointer); CHECK_I32(edgeList); CHECK_I32(backEdgeMask); CHECK_I32(node_degs);
  CHECK_BOOL(src_mask); CHECK_BOOL(ngh_mask);
  const bool is_last = layer == num_layers;
  TORCH_CHECK(is_last || ngh_mask.numel() == src_mask.numel(),
              "ngh_mask must cover every vertex before the last preparation step");
  TORCH_CHECK(partPointer.numel() == id.numel() + 1 || id.numel() == 0,
              "partPointer must have one more entry than id");
  c10::cuda::CUDAGuard guard(id.device());
  ScopedTime t(4);
  epp_check(eppgcn_mask_forward(id.data_ptr<int>(), partPointer.data_ptr<int>(), edgeList.data_ptr<int>(),
                                reinterpret_cast<const unsigned char *>(src_mask.data_ptr<bool>()),
                                ngh_mask.numel() ? reinterpret_cast<unsigned char *>(ngh_mask.data_ptr<bool>())
                                                 : nullptr,
                                backEdgeMask.data_ptr<int>(), node_degs.data_ptr<int>(),
                                static_cast<int>(id.numel()), is_last ? 1 : 0, 0, blockx, blocky,
                                current_stream()),
            "eppgcn_mask_forward");
}

// ours_backward(d_output, X, W, id, partPointer, edgeList, degrees, partSize,
//               numParts, layer, blockx, blocky) -> [d_input, d_weight]
// EPPGCN.cpp:157-184, EPPGCN_kernel.cu:547-624.
std::vector<torch::Tensor> ours_backward_impl(torch::Tensor d_output, torch::Tensor X, torch::Tensor W,
                                              torch::Tensor id, torch::Tensor partPointer, torch::Tensor edgeList,
                                              torch::Tensor degrees, int partSize, int numParts, int layer,
                                              int blockx, int blocky, bool need_d_input) {
  CHECK_INPUT(d_output); CHECK_INPUT(X); CHECK_INPUT(W); CHECK_INPUT(id); CHECK_INPUT(partPointer);
  CHECK_INPUT(edgeList); CHECK_INPUT(degrees);
  CHECK_F32(d_output); CHECK_F32(X); CHECK_F32(W); CHECK_F32(degrees);
  CHECK_I32(id); CHECK_I32(partPointer); CHECK_I32(edgeList);
  TORCH_CHECK(numParts >= 0 && (numParts == 0 || numParts < partPointer.numel()),
              "partPointer must hold numParts + 1 entries");
  c10::cuda::CUDAGuard guard(d_output.device());
  const int64_t n = d_output.size(0), d = d_output.size(1);
  torch::Tensor d_input_prime;
  const eppgcn_tile_plan *plan = nullptr;
  if (plans_enabled() && n > 0) {
    ScopedTime t(2, layer);
    plan = backward_plan(id, partPointer, edgeList, numParts, n);
    d_input_prime = aggregate_planned(plan, pack_scaled(plan, d_output, degrees), degrees, n);
  } else {
    d_input_prime = at::empty({n, d}, d_output.options());
    ScopedTime t(2, layer);
    epp_check(eppgcn_spmm_backward_compacted(d_input_prime.data_ptr<float>(), 0, d_output.data_ptr<float>(), d,
                                             id.data_ptr<int>(), partPointer.data_ptr<int>(),
                                             edgeList.data_ptr<int>(), degrees.data_ptr<float>(),
                                             degrees.data_ptr<float>(), static_cast<int>(n), static_cast<int>(d),
                                             numParts, partSize, blockx, blocky, current_stream()),
              "eppgcn_spmm_backward_compacted");
  }
  ScopedTime t(3);
  return backward_update(d_input_prime, X, W, plan, need_d_input);
}

std::vector<torch::Tensor> ours_backward(torch::Tensor d_output, torch::Tensor X, torch::Tensor W,
                                         torch::Tensor id, torch::Tensor partPointer, torch::Tensor edgeList,
                                         torch::Tensor degrees, int partSize, int numParts, int layer,
                                         int blockx, int blocky) {
  return ours_backward_impl(d_output, X, W, id, partPointer, edgeList, degrees, partSize, numParts, layer, blockx,
                            blocky, true);
}

// ours_backward for a layer whose input needs no gradient (the first layer of a model: its input is
// the feature matrix): returns [empty, d_weight] and skips the d' @ W^T product and its [N, Din] result.
// Not in the reference, which computes that product for every layer.
std::vector<torch::Tensor> ours_backward_weight_only(torch::Tensor d_output, torch::Tensor X, torch::Tensor W,
                                                     torch::Tensor id, torch::Tensor partPointer,
                                                     torch::Tensor edgeList, torch::Tensor degrees, int partSize,
                                                     int numParts, int layer, int blockx, int blocky) {
  return ours_backward_impl(d_output, X, W, id, partPointer, edgeList, degrees, partSize, numParts, layer, blockx,
                            blocky, false);
}

// build_part(partSize, indptr) -> [partPtr, part2Node]      EPPGCN.cpp:186-227
std::vector<torch::Tensor> build_part(int partSize, torch::Tensor indptr) {
  CHECK_I32(indptr);
  if (indptr.is_cuda()) {
    // Beyond the reference (its build_part takes a CPU tensor only): a row pointer that already
    // lives on the device is partitioned there, and the groups come back as CUDA tensors.
    TORCH_CHECK(indptr.dim() == 1 && indptr.numel() >= 1, "indptr must be a 1-D tensor of num_nodes + 1 entries");
    TORCH_CHECK(partSize >= 1, "partSize must be >= 1, got ", partSize);
    c10::cuda::CUDAGuard guard(indptr.device());
    auto ip = indptr.contiguous();
    const int n = static_cast<int>(ip.numel() - 1);
    const int64_t edges = n > 0 ? ip[n].item<int>() : 0;
    const int64_t cap = edges / partSize + n + 1;
    TORCH_CHECK(cap + 1 < (1LL << 31), "group count exceeds int32");
    auto partPtr = at::empty({cap + 1}, ip.options());
    auto part2Node = at::empty({cap}, ip.options());
    const size_t bytes = eppgcn_build_part_scratch_bytes(n);
    auto scratch = at::empty({static_cast<int64_t>((bytes + 7) / 8)}, ip.options().dtype(at::kLong));
    auto counter = at::empty({2}, ip.options());
    for (int mode = 0; mode < 2; ++mode) {
      epp_check(eppgcn_build_part(ip.data_ptr<int>(), n, partSize, partPtr.data_ptr<int>(), static_cast<int>(cap + 1),
                                  part2Node.data_ptr<int>(), static_cast<int>(cap), scratch.data_ptr(), bytes,
                                  counter.data_ptr<int>(), counter.data_ptr<int>() + 1, mode, current_stream()),
                "eppgcn_build_part");
      auto host = counter.cpu();
      const int parts = host.data_ptr<int>()[0], status = host.data_ptr<int>()[1];
      if (status == EPP_OK) return {partPtr.narrow(0, 0, parts + 1).clone(), part2Node.narrow(0, 0, parts).clone()};
      if (mode == 1) epp_check(status, "eppgcn_build_part");      // mode 0 ran out of its bounded wait: repeat without waiting
    }
  }
  TORCH_CHECK(indptr.dim() == 1 && indptr.numel() >= 1, "indptr must be a 1-D tensor of num_nodes + 1 entries");
  auto ip = indptr.contiguous();
  const int n = static_cast<int>(ip.numel() - 1);
  long long total = 0;
  epp_check(eppgcn_build_part_host(partSize, ip.data_ptr<int>(), n, nullptr, nullptr, &total),
            "eppgcn_build_part_host");
  auto opts = at::TensorOptions().dtype(at::kInt).device(at::kCPU);
  auto partPtr = at::empty({total + 1}, opts);
  auto part2Node = at::empty({total}, opts);
  epp_check(eppgcn_build_part_host(partSize, ip.data_ptr<int>(), n, partPtr.data_ptr<int>(),
                                   part2Node.data_ptr<int>(), &total),
            "eppgcn_build_part_host");
  return {partPtr, part2Node};
}

struct Compacted {
  torch::Tensor id, edge_list;
  int valid_len;
};

Compacted compact_edges(const torch::Tensor &edge_mask, const torch::Tensor &column_index) {
  CHECK_INPUT(edge_mask); CHECK_INPUT(column_index);
  CHECK_I32(edge_mask); CHECK_I32(column_index);
  TORCH_CHECK(edge_mask.numel() == column_index.numel(), "edge_mask and column_index must have equal length");
  TORCH_CHECK(edge_mask.numel() < (1LL << 31), "edge count exceeds int32");
  c10::cuda::CUDAGuard guard(edge_mask.device());
  const int length = static_cast<int>(edge_mask.numel());
  auto id = at::empty_like(edge_mask);
  auto edge_list = at::empty_like(column_index);
  const size_t bytes = eppgcn_compact_scratch_bytes(length);
  auto scratch = at::empty({static_cast<int64_t>(bytes)}, edge_mask.options().dtype(at::kByte));
  auto counter = at::empty({2}, edge_mask.options());
  epp_check(eppgcn_compact_mask(edge_mask.data_ptr<int>(), column_index.data_ptr<int>(), id.data_ptr<int>(),
                                edge_list.data_ptr<int>(), length, scratch.data_ptr(), bytes,
                                counter.data_ptr<int>(), counter.data_ptr<int>() + 1, 0, current_stream()),
            "eppgcn_compact_mask");
  auto host = counter.cpu();
  if (host.data_ptr<int>()[1] == EPP_ERR_SCAN_TIMEOUT) {   // bounded wait ran out: redo without waiting
    epp_check(eppgcn_compact_mask(edge_mask.data_ptr<int>(), column_index.data_ptr<int>(), id.data_ptr<int>(),
                                  edge_list.data_ptr<int>(), length, scratch.data_ptr(), bytes,
                                  counter.data_ptr<int>(), counter.data_ptr<int>() + 1, 1, current_stream()),
              "eppgcn_compact_mask");
    host = counter.cpu();
  }
  epp_check(host.data_ptr<int>()[1], "eppgcn_compact_mask");
  return {id, edge_list, host.data_ptr<int>()[0]};
}

struct Split {
  torch::Tensor part_pointer;
  int num_parts;
};

Split split_parts(const torch::Tensor &node_deg, int num_edges, int back_part_size) {
  CHECK_INPUT(node_deg);
  CHECK_I32(node_deg);
  TORCH_CHECK(num_edges >= 0, "num_edges must be non-negative");
  TORCH_CHECK(back_part_size >= 1, "back_part_size must be >= 1, got ", back_part_size);
  c10::cuda::CUDAGuard guard(node_deg.device());
  const int n = static_cast<int>(node_deg.numel());
  // One entry more than the reference allocates (EPPGCN.cpp:335-336), so the
  // closing pointer exists even when every part holds a single edge.
  const int out_len = num_edges + 1;
  auto part_pointer = at::empty({out_len}, node_deg.options());
  const size_t bytes = eppgcn_split_scratch_bytes(n);
  auto scratch = at::empty({static_cast<int64_t>(bytes)}, node_deg.options().dtype(at::kByte));
  auto counter = at::empty({2}, node_deg.options());
  for (int mode = 0; mode < 2; ++mode) {
    epp_check(eppgcn_split_parts(node_deg.data_ptr<int>(), n, back_part_size,
                                 part_pointer.data_ptr<int>(), out_len,
                                 scratch.data_ptr(), bytes, counter.data_ptr<int>(), counter.data_ptr<int>() + 1,
                                 mode, current_stream()),
              "eppgcn_split_parts");
    auto host = counter.cpu();
    if (host.data_ptr<int>()[1] == EPP_OK) return {part_pointer, host.data_ptr<int>()[0]};
    if (mode == 1) epp_check(host.data_ptr<int>()[1], "eppgcn_split_parts");
  }
  return {part_pointer, 0};
}

int count_active(const torch::Tensor &node_deg) {
  CHECK_INPUT(node_deg);
  CHECK_I32(node_deg);
  c10::cuda::CUDAGuard guard(node_deg.device());
  auto counter = at::empty({1}, node_deg.options());
  epp_check(eppgcn_count_nonzero(node_deg.data_ptr<int>(), static_cast<int>(node_deg.numel()),
                                 counter.data_ptr<int>(), current_stream()),
            "eppgcn_count_nonzero");
  return counter.item<int>();
}

// compact_back_edge(edge_mask, column_index) -> [id, edge_list, info]   EPPGCN.cpp:282-296
std::vector<torch::Tensor> compact_back_edge(torch::Tensor edge_mask, torch::Tensor column_index) {
  Compacted c = compact_edges(edge_mask, column_index);
  auto info = at::zeros({1}, at::TensorOptions().dtype(at::kDouble));
  info.data_ptr<double>()[0] = c.valid_len;
  return {c.id, c.edge_list, info};
}

// get_map_back_part_size(node_deg, valid_len) -> int   EPPGCN.cpp:298-325
// Unclamped, as in the reference: the value can be zero or negative on large
// graphs and the caller has to clamp it before split_back_part.
int get_map_back_part_size(torch::Tensor node_deg, int valid_len) {
  int ps = 0;
  epp_check(eppgcn_map_back_part_size(count_active(node_deg), valid_len, &ps), "eppgcn_map_back_part_size");
  return ps;
}

// split_back_part(node_deg, num_edges, back_part_size) -> [part_pointer, info]   EPPGCN.cpp:327-346
std::vector<torch::Tensor> split_back_part(torch::Tensor node_deg, int num_edges, int back_part_size) {
  Split s = split_parts(node_deg, num_edges, back_part_size);
  auto info = at::zeros({1}, at::TensorOptions().dtype(at::kInt));
  info.data_ptr<int>()[0] = s.num_parts;
  return {s.part_pointer, info};
}

// build_back_part(edge_mask, column_index, node_deg, back_part_size, dim)
//   -> [id, edge_list, part_pointer, info(float[2]) = {part size, num_parts}]   EPPGCN.cpp:229-280
std::vector<torch::Tensor> build_back_part(torch::Tensor edge_mask, torch::Tensor column_index,
                                           torch::Tensor node_deg, int back_part_size, int dim) {
  (void)dim;
  Compacted c = compact_edges(edge_mask, column_index);
  if (back_part_size == 0) {
    epp_check(eppgcn_bucket_back_part_size(count_active(node_deg), c.valid_len, &back_part_size),
              "eppgcn_bucket_back_part_size");
    TORCH_CHECK(back_part_size >= 1, "average active degree is 512 or more: pass an explicit back_part_size");
  }
  Split s = split_parts(node_deg, static_cast<int>(column_index.numel()), back_part_size);
  auto info = at::zeros({2}, at::TensorOptions().dtype(at::kDouble));
  info.data_ptr<double>()[0] = back_part_size;
  info.data_ptr<double>()[1] = s.num_parts;
  return {c.id, c.edge_list, s.part_pointer, info};
}

// get_ginfo(node_deg, valid_len) -> float32[10]   EPPGCN.cpp:348-386
torch::Tensor get_ginfo(torch::Tensor node_deg, int valid_len) {
  TORCH_CHECK(!node_deg.is_cuda(), "node_deg must be a CPU tensor");
  CHECK_I32(node_deg);
  auto nd = node_deg.contiguous();
  auto re = at::zeros({10}, at::TensorOptions().dtype(at::kFloat));
  epp_check(eppgcn_get_ginfo_host(nd.data_ptr<int>(), static_cast<int>(nd.numel()), valid_len,
                                  re.data_ptr<float>()),
            "eppgcn_get_ginfo_host");
  return re;
}

// Extras beside the reference's twelve functions: the plans the operators keep.
void clear_plans() { plan_cache().clear(); }
int64_t num_plans() { return static_cast<int64_t>(plan_cache().size()); }

void print_time() { epp_check(eppgcn_print_time(), "eppgcn_print_time"); }
void clear_time() { epp_check(eppgcn_clear_time(), "eppgcn_clear_time"); }

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("forward", &spmm_forward, "GCN layer forward: X @ W, then neighbour-group aggregation (CUDA)");
  m.def("backward", &spmm_backward, "GCN layer backward over the whole graph (CUDA)");
  m.def("mask_forward", &mask_forward, "execution-path marking for one preparation step (CUDA)");
  m.def("ours_backward", &ours_backward, "GCN layer backward over the prepared execution path (CUDA)");
  m.def("print_time", &print_time, "print accumulated kernel times");
  m.def("clear_time", &clear_time, "reset accumulated kernel times");
  m.def("build_part", &build_part, "neighbour-group partition (CPU)");
  m.def("build_back_part", &build_back_part, "compaction + part-size rule + splitting in one call (CUDA)");
  m.def("compact_back_edge", &compact_back_edge, "stable compaction of the marked edges (CUDA)");
  m.def("get_map_back_part_size", &get_map_back_part_size, "regression rule for the backward part size (CUDA)");
  m.def("split_back_part", &split_back_part, "split active rows into backward parts (CUDA)");
  m.def("get_ginfo", &get_ginfo, "degree histogram features (CPU)");
  m.def("ours_backward_weight_only", &ours_backward_weight_only,
        "ours_backward without the input gradient: [empty, d_weight] (not in the reference)");
  m.def("clear_plans", &clear_plans, "drop the aggregation plans the operators keep (not in the reference)");
  m.def("num_plans", &num_plans, "number of aggregation plans currently kept (not in the reference)");
}
