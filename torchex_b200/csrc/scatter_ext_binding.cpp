// Torch extension module `scatter_ext`: tensors in, the C ABI of
// include/texb_scatter.h underneath.
//
// The first three functions are the whole interface of TorchEx's own module of
// that name (torchex/src/scatter/scatter.cpp:20-70): sum(feats, preSum, out,
// max_cnt), max(feats, preSum, out, arg, max_cnt) and getPreSum(unq_inv, preSum),
// with the same argument lists, the same in-place outputs and the same
// "must be a CUDAtensor" / "must be contiguous" checks, so TorchEx's
// operator_py/scatter_op.py runs on this module unchanged.  Unlike the reference
// binding, each call also checks dtypes and shapes, runs on the tensor's own device
// and on torch's current stream, takes its scratch from torch's caching allocator
// and turns a failed launch into a RuntimeError.
//
// The rest serves torchex_b200.operator_py: a Plan object (the device arrays of a
// ScatterData plus what the host knows about them) and one call per operator that
// allocates the outputs, picks the kernel path and launches -- a single trip from
// Python per reduction.

#include <torch/extension.h>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <tuple>
#include <vector>

#include "texb_scatter.h"

namespace {

#define TEXB_CHECK_CUDA(x) TORCH_CHECK((x).device().is_cuda(), #x, " must be a CUDAtensor ")
#define TEXB_CHECK_CONTIGUOUS(x) TORCH_CHECK((x).is_contiguous(), #x, " must be contiguous ")
#define TEXB_CHECK_INPUT(x) \
  TEXB_CHECK_CUDA(x);       \
  TEXB_CHECK_CONTIGUOUS(x)
#define TEXB_CHECK_DTYPE(x, t) \
  TORCH_CHECK((x).scalar_type() == (t), #x, " must have dtype ", (t), ", got ", (x).scalar_type())

void check_status(int status, const char* what) {
  TORCH_CHECK(status == TEXB_OK, what, " failed with status ", status, ": ", texb_last_error());
}

void* stream_of(const at::Tensor& t) {
  return static_cast<void*>(at::cuda::getCurrentCUDAStream(t.get_device()).stream());
}

at::Tensor scratch(size_t bytes, const at::Tensor& like) {
  return at::empty({static_cast<int64_t>(bytes > 0 ? bytes : 1)}, like.options().dtype(at::kByte));
}

// ---- the reference's three functions ------------------------------------------------

void scatter_sum_gpu(at::Tensor feats, at::Tensor preSum, at::Tensor out, int max_cnt) {
  TEXB_CHECK_INPUT(feats);
  TEXB_CHECK_INPUT(preSum);
  TEXB_CHECK_INPUT(out);
  TEXB_CHECK_DTYPE(feats, at::kFloat);
  TEXB_CHECK_DTYPE(preSum, at::kInt);
  TEXB_CHECK_DTYPE(out, at::kFloat);
  TORCH_CHECK(feats.dim() == 2 && out.dim() == 2, "feats and out must be [rows, channel]");
  const int64_t n = feats.size(0), c = feats.size(1), m = out.size(0);
  TORCH_CHECK(preSum.numel() == m + 1 && out.size(1) == c,
              "scatter_ext.sum: preSum must have out.size(0) + 1 entries and out the channel count of feats");
  const c10::cuda::CUDAGuard guard(feats.device());
  at::Tensor ws;
  void* ws_ptr = nullptr;
  size_t ws_bytes = 0;
  if (!(max_cnt > 0 && texb_segment_reduce_small_ok(n, int(c), max_cnt))) {
    ws_bytes = texb_scatter_compat_workspace_bytes(n, int(c));
    ws = scratch(ws_bytes, feats);
    ws_ptr = ws.data_ptr();
  }
  check_status(texb_scatter_sum(feats.data_ptr<float>(), preSum.data_ptr<int>(), out.data_ptr<float>(), int(c),
                                int(m), max_cnt, n, ws_ptr, ws_bytes, stream_of(feats)),
               "texb_scatter_sum");
}

void scatter_max_gpu(at::Tensor feats, at::Tensor preSum, at::Tensor out, at::Tensor arg, int max_cnt) {
  TEXB_CHECK_INPUT(feats);
  TEXB_CHECK_INPUT(preSum);
  TEXB_CHECK_INPUT(out);
  TEXB_CHECK_INPUT(arg);
  TEXB_CHECK_DTYPE(feats, at::kFloat);
  TEXB_CHECK_DTYPE(preSum, at::kInt);
  TEXB_CHECK_DTYPE(out, at::kFloat);
  TEXB_CHECK_DTYPE(arg, at::kInt);
  TORCH_CHECK(feats.dim() == 2 && out.dim() == 2, "feats and out must be [rows, channel]");
  const int64_t n = feats.size(0), c = feats.size(1), m = out.size(0);
  TORCH_CHECK(preSum.numel() == m + 1 && out.size(1) == c && arg.sizes() == out.sizes(),
              "scatter_ext.max: preSum must have out.size(0) + 1 entries and out / arg the shape [num_unq, channel]");
  const c10::cuda::CUDAGuard guard(feats.device());
  at::Tensor ws;
  void* ws_ptr = nullptr;
  size_t ws_bytes = 0;
  if (!(max_cnt > 0 && texb_segment_reduce_small_ok(n, int(c), max_cnt))) {
    ws_bytes = texb_scatter_compat_workspace_bytes(n, int(c));
    ws = scratch(ws_bytes, feats);
    ws_ptr = ws.data_ptr();
  }
  check_status(texb_scatter_max(feats.data_ptr<float>(), preSum.data_ptr<int>(), out.data_ptr<float>(),
                                arg.data_ptr<int>(), int(c), int(m), max_cnt, n, ws_ptr, ws_bytes,
                                stream_of(feats)),
               "texb_scatter_max");
}

void get_pre_sum_gpu(at::Tensor unq_inv, at::Tensor preSum) {
  TEXB_CHECK_INPUT(unq_inv);
  TEXB_CHECK_INPUT(preSum);
  TEXB_CHECK_DTYPE(unq_inv, at::kInt);
  TEXB_CHECK_DTYPE(preSum, at::kInt);
  TORCH_CHECK(preSum.numel() >= 1, "preSum needs at least one entry");
  const c10::cuda::CUDAGuard guard(unq_inv.device());
  check_status(texb_get_pre_sum(unq_inv.data_ptr<int>(), preSum.data_ptr<int>(), unq_inv.numel(),
                                preSum.numel() - 1, stream_of(unq_inv)),
               "texb_get_pre_sum");
}

// ---- plan-based operators ---------------------------------------------------------------

struct Plan {
  at::Tensor sid;      // int32 [n]: segment id at each segment-sorted position
  at::Tensor perm;     // int32 [n]: feats row at that position; undefined when the ids arrived sorted
  at::Tensor offsets;  // int32 [m + 1]: TorchEx's preSum
  at::Tensor balance;  // int32 [K + 1]: cost-balanced cut points of the sorted rows
  int64_t num_total = 0, num_segments = 0;
  int64_t max_cnt = -1;    // rows of the largest segment, -1 while the host does not know it
  bool has_empty = true;   // false only once the host knows that every segment has rows
  bool settled = false;    // the host has synchronised with the stream since the arrays were built
  bool no_split = false;   // every cut of the balance table is a segment start (short segments only)
  struct Scratch {
    int64_t channels;
    int slot;  // 0: single calls; k: the k-th reduction of a sequence; -1: the two-output operator
    void* stream;
    at::Tensor buffer;
  };
  std::vector<Scratch> scratch_cache;  // one buffer per (channel count, operator kind, stream)

  int flags() const {
    return (has_empty || num_total == 0 ? TEXB_PLAN_HAS_EMPTY : 0) | (settled ? TEXB_PLAN_SETTLED : 0) |
           (no_split ? TEXB_PLAN_NO_SPLIT : 0);
  }
  const int32_t* perm_ptr() const { return perm.defined() ? perm.data_ptr<int>() : nullptr; }

  // Calls on one stream are ordered, so they can share a buffer; another stream gets its own.
  at::Tensor& workspace(int64_t channels, int slot, void* stream, size_t bytes) {
    for (auto& s : scratch_cache)
      if (s.channels == channels && s.slot == slot && s.stream == stream) {
        if (size_t(s.buffer.numel()) < bytes) s.buffer = scratch(bytes, sid);
        return s.buffer;
      }
    scratch_cache.push_back({channels, slot, stream, scratch(bytes, sid)});
    return scratch_cache.back().buffer;
  }
};

Plan make_plan(at::Tensor sid, c10::optional<at::Tensor> perm, at::Tensor offsets, at::Tensor balance,
               int64_t num_segments, bool has_empty, int64_t max_cnt, bool settled) {
  TEXB_CHECK_INPUT(sid);
  TEXB_CHECK_INPUT(offsets);
  TEXB_CHECK_INPUT(balance);
  TEXB_CHECK_DTYPE(sid, at::kInt);
  TEXB_CHECK_DTYPE(offsets, at::kInt);
  TEXB_CHECK_DTYPE(balance, at::kInt);
  TORCH_CHECK(offsets.numel() == num_segments + 1, "offsets must have num_segments + 1 entries");
  TORCH_CHECK(balance.numel() >= 2, "balance needs at least two entries");
  Plan p;
  p.sid = sid;
  if (perm.has_value() && perm->defined()) {
    TEXB_CHECK_INPUT((*perm));
    TEXB_CHECK_DTYPE((*perm), at::kInt);
    TORCH_CHECK(perm->numel() == sid.numel(), "perm and sid differ in length");
    p.perm = *perm;
  }
  p.offsets = offsets;
  p.balance = balance;
  p.num_total = sid.numel();
  p.num_segments = num_segments;
  p.has_empty = has_empty;
  p.max_cnt = max_cnt;
  p.settled = settled;
  return p;
}

// Builds the segment plan of ScatterData in one call: inspection of the ids (the one
// synchronisation with the device: sortedness, range, run count), then -- if the ids fit
// the `m` segments -- the sort (skipped for sorted ids), offsets, statistics and balance
// table, and an asynchronous copy of the statistics to pinned host memory.  Returns
//   (is_sorted, id_min, id_max, runs, m, sid, perm | None, offsets, balance, stats_host)
// with sid .. stats_host None when the ids lie outside [0, m) (the caller raises).
// m < 0: take the largest id + 1.  Replaces the constructor of the reference class and
// its getPreSum call (torchex/operator_py/scatter_op.py:8-21, 114-135).
py::tuple build_plan(const at::Tensor& ids_in, int64_t m, int64_t balance_pieces) {
  TORCH_CHECK(ids_in.device().is_cuda(), "unq_inv must be a CUDAtensor");
  TORCH_CHECK(ids_in.scalar_type() == at::kInt || ids_in.scalar_type() == at::kLong, "ids must be int32 or int64");
  TORCH_CHECK(balance_pieces >= 1, "balance_pieces must be positive");
  const at::Tensor ids = ids_in.reshape({-1}).contiguous();
  const int64_t n = ids.numel();
  const int id_bytes = int(ids.element_size());
  const c10::cuda::CUDAGuard guard(ids.device());
  void* stream = stream_of(ids);
  const auto i32 = ids.options().dtype(at::kInt);
  at::Tensor stats = at::empty({4}, i32);
  check_status(texb_ids_inspect(ids.data_ptr(), id_bytes, n, stats.data_ptr<int>(), stream), "texb_ids_inspect");
  const at::Tensor h = stats.to(at::kCPU);  // the one synchronisation
  const int32_t* hs = h.data_ptr<int>();
  const bool is_sorted = hs[0] != 0;
  const int64_t id_min = hs[1], id_max = hs[2], runs = hs[3];
  if (m < 0) m = n > 0 ? id_max + 1 : 0;
  if (n > 0 && (id_min < 0 || id_max >= m))
    return py::make_tuple(is_sorted, id_min, id_max, runs, m, py::none(), py::none(), py::none(), py::none(), py::none());
  at::Tensor offsets = at::empty({m + 1}, i32);
  at::Tensor plan_stats = at::empty({4}, i32);
  at::Tensor sid, perm;
  if (is_sorted) {
    sid = ids.scalar_type() == at::kInt ? ids : at::empty({n}, i32);
  } else {
    sid = at::empty({n}, i32);
    perm = at::empty({n}, i32);
  }
  const size_t ws_bytes = texb_plan_workspace_bytes(n, m, is_sorted ? 1 : 0);
  at::Tensor ws = scratch(ws_bytes, ids);
  check_status(texb_plan_build(ids.data_ptr(), id_bytes, n, m, is_sorted ? 1 : 0, sid.data_ptr<int>(),
                               perm.defined() ? perm.data_ptr<int>() : nullptr, offsets.data_ptr<int>(),
                               plan_stats.data_ptr<int>(), ws.data_ptr(), size_t(ws.numel()), stream),
               "texb_plan_build");
  at::Tensor balance = at::empty({balance_pieces + 1}, i32);
  check_status(texb_plan_balance(sid.data_ptr<int>(), n, balance.data_ptr<int>(), int(balance.numel()),
                                 plan_stats.data_ptr<int>(), stream),
               "texb_plan_balance");
  at::Tensor stats_host = at::empty({4}, at::TensorOptions().dtype(at::kInt).pinned_memory(true));
  stats_host.copy_(plan_stats, /*non_blocking=*/true);
  return py::make_tuple(is_sorted, id_min, id_max, runs, m, sid, perm.defined() ? py::cast(perm) : py::object(py::none()),
                        offsets, balance, stats_host);
}

// feats as the kernels take them: contiguous fp32, or bf16 where the bf16 kernel covers the shape.
at::Tensor prepare_feats(const Plan& p, const at::Tensor& feats, bool pair) {
  TORCH_CHECK(feats.device().is_cuda(), "feats must be a CUDAtensor ");
  TORCH_CHECK(feats.scalar_type() == at::kFloat || feats.scalar_type() == at::kBFloat16,
              "feats must be float32 (or bfloat16), got ", feats.scalar_type());
  TORCH_CHECK(feats.dim() == 2, "feats must be [num_total, channel]");
  TORCH_CHECK(feats.size(0) == p.num_total, "feats has ", feats.size(0), " rows but ScatterData was built for ",
              p.num_total);
  TORCH_CHECK(feats.device() == p.sid.device(), "feats and ScatterData live on different devices");
  TORCH_CHECK(feats.size(1) >= 1, "feats needs at least one channel");
  at::Tensor f = feats.contiguous();
  if (f.scalar_type() == at::kBFloat16) {
    const int64_t c = f.size(1);
    const bool covered = c % 8 == 0 && (pair ? c == 128 : c >= 128) &&
                         reinterpret_cast<uintptr_t>(f.data_ptr()) % 16 == 0;
    if (!covered) f = f.to(at::kFloat);  // the bf16 kernel covers wide, aligned rows; others are widened first
  }
  return f;
}

// An output the caller provides (e.g. a buffer that other processes map) instead of a fresh tensor.
at::Tensor output_rows(const c10::optional<at::Tensor>& given, const at::Tensor& feats, int64_t m, int64_t c,
                       at::ScalarType dtype, const char* name) {
  if (!given.has_value() || !given->defined()) return at::empty({m, c}, feats.options().dtype(dtype));
  const at::Tensor& t = *given;
  TORCH_CHECK(t.device() == feats.device(), name, " must be on the device of feats");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous ");
  TORCH_CHECK(t.scalar_type() == dtype, name, " must have dtype ", dtype, ", got ", t.scalar_type());
  TORCH_CHECK(t.dim() == 2 && t.size(0) == m && t.size(1) == c, name, " must be [num_unq, channel]");
  return t;
}

std::tuple<at::Tensor, c10::optional<at::Tensor>> reduce(Plan& p, int op, const at::Tensor& feats_in,
                                                         int64_t arg_base, c10::optional<at::Tensor> out_given,
                                                         c10::optional<at::Tensor> arg_given) {
  TORCH_CHECK(op == TEXB_OP_SUM || op == TEXB_OP_MEAN || op == TEXB_OP_MAX, "unknown reduce op ", op);
  const at::Tensor feats = prepare_feats(p, feats_in, false);
  const int64_t n = feats.size(0), c = feats.size(1), m = p.num_segments;
  const c10::cuda::CUDAGuard guard(feats.device());
  void* stream = stream_of(feats);
  at::Tensor out = output_rows(out_given, feats, m, c, at::kFloat, "out");
  c10::optional<at::Tensor> arg;
  int32_t* arg_ptr = nullptr;
  if (op == TEXB_OP_MAX) {
    arg = output_rows(arg_given, feats, m, c, at::kInt, "arg");
    arg_ptr = arg->data_ptr<int>();
  }
  const bool bf16 = feats.scalar_type() == at::kBFloat16;
  if (!bf16 && texb_segment_reduce_small_ok(n, int(c), p.max_cnt)) {
    check_status(texb_segment_reduce_small(op, feats.data_ptr<float>(), p.offsets.data_ptr<int>(), p.perm_ptr(), n,
                                           int(c), m, out.data_ptr<float>(), arg_ptr, int32_t(arg_base), stream),
                 "texb_segment_reduce_small");
    return {out, arg};
  }
  at::Tensor& ws = p.workspace(c, 0, stream, texb_reduce_workspace_bytes(n, int(c)));
  if (bf16) {
    check_status(texb_segment_reduce_bf16(op, feats.data_ptr(), p.sid.data_ptr<int>(), p.perm_ptr(),
                                          p.offsets.data_ptr<int>(), p.flags(), p.balance.data_ptr<int>(),
                                          int(p.balance.numel()), n, int(c), m, out.data_ptr<float>(), arg_ptr,
                                          int32_t(arg_base), ws.data_ptr(), size_t(ws.numel()), stream),
                 "texb_segment_reduce_bf16");
  } else {
    check_status(texb_segment_reduce(op, feats.data_ptr<float>(), p.sid.data_ptr<int>(), p.perm_ptr(),
                                     p.offsets.data_ptr<int>(), p.flags(), p.balance.data_ptr<int>(),
                                     int(p.balance.numel()), n, int(c), m, out.data_ptr<float>(), arg_ptr,
                                     int32_t(arg_base), ws.data_ptr(), size_t(ws.numel()), stream),
                 "texb_segment_reduce");
  }
  return {out, arg};
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> reduce_pair(Plan& p, int op, const at::Tensor& feats_in,
                                                           int64_t arg_base, c10::optional<at::Tensor> sum_given,
                                                           c10::optional<at::Tensor> max_given,
                                                           c10::optional<at::Tensor> arg_given) {
  TORCH_CHECK(op == TEXB_OP_SUM || op == TEXB_OP_MEAN, "the two-output reduction pairs the maximum with sum or mean");
  const at::Tensor feats = prepare_feats(p, feats_in, true);
  const int64_t n = feats.size(0), c = feats.size(1), m = p.num_segments;
  const c10::cuda::CUDAGuard guard(feats.device());
  void* stream = stream_of(feats);
  at::Tensor out_sum = output_rows(sum_given, feats, m, c, at::kFloat, "out_sum");
  at::Tensor out_max = output_rows(max_given, feats, m, c, at::kFloat, "out_max");
  at::Tensor arg = output_rows(arg_given, feats, m, c, at::kInt, "arg");
  at::Tensor& ws = p.workspace(c, -1, stream, texb_reduce_pair_workspace_bytes(n, int(c)));
  check_status(texb_segment_reduce_pair(op, feats.data_ptr(), int(feats.element_size()), p.sid.data_ptr<int>(),
                                        p.perm_ptr(), p.offsets.data_ptr<int>(), p.flags(),
                                        p.balance.data_ptr<int>(), int(p.balance.numel()), n, int(c), m,
                                        out_sum.data_ptr<float>(), out_max.data_ptr<float>(), arg.data_ptr<int>(),
                                        int32_t(arg_base), ws.data_ptr(), size_t(ws.numel()), stream),
               "texb_segment_reduce_pair");
  return {out_sum, out_max, arg};
}

// Several reductions of the same rows, issued back to back as one sequence
// (TEXB_SEQUENCE_FIRST / TEXB_SEQUENCE_NEXT): the second and later ones do not wait for the
// stream at their start, so each takes over the SMs as the one before it drains.  Every
// reduction has its own outputs and its own workspace.  Returns one (out, arg | None) per op.
std::vector<std::tuple<at::Tensor, c10::optional<at::Tensor>>> reduce_sequence(Plan& p, const std::vector<int>& ops,
                                                                               const at::Tensor& feats_in,
                                                                               int64_t arg_base) {
  const at::Tensor feats = prepare_feats(p, feats_in, false);
  const int64_t n = feats.size(0), c = feats.size(1), m = p.num_segments;
  const bool bf16 = feats.scalar_type() == at::kBFloat16;
  std::vector<std::tuple<at::Tensor, c10::optional<at::Tensor>>> results;
  // The one-launch kernel for small inputs, a plan the host does not yet know to be complete,
  // or a plan that may have empty segments (their fill is a launch of its own between the
  // reductions): plain calls, one after the other.
  if ((!bf16 && texb_segment_reduce_small_ok(n, int(c), p.max_cnt)) || !p.settled || p.has_empty || n == 0) {
    for (int op : ops) results.push_back(reduce(p, op, feats, arg_base, c10::nullopt, c10::nullopt));
    return results;
  }
  const c10::cuda::CUDAGuard guard(feats.device());
  void* stream = stream_of(feats);
  int k = 0;
  for (int op : ops) {
    TORCH_CHECK(op == TEXB_OP_SUM || op == TEXB_OP_MEAN || op == TEXB_OP_MAX, "unknown reduce op ", op);
    at::Tensor out = at::empty({m, c}, feats.options().dtype(at::kFloat));
    c10::optional<at::Tensor> arg;
    int32_t* arg_ptr = nullptr;
    if (op == TEXB_OP_MAX) {
      arg = at::empty({m, c}, feats.options().dtype(at::kInt));
      arg_ptr = arg->data_ptr<int>();
    }
    at::Tensor& ws = p.workspace(c, k + 1, stream, texb_reduce_workspace_bytes(n, int(c)));
    const int flags = p.flags() | (k == 0 ? TEXB_SEQUENCE_FIRST : TEXB_SEQUENCE_NEXT);
    const int st = bf16
        ? texb_segment_reduce_bf16(op, feats.data_ptr(), p.sid.data_ptr<int>(), p.perm_ptr(), p.offsets.data_ptr<int>(),
                                   flags, p.balance.data_ptr<int>(), int(p.balance.numel()), n, int(c), m,
                                   out.data_ptr<float>(), arg_ptr, int32_t(arg_base), ws.data_ptr(), size_t(ws.numel()),
                                   stream)
        : texb_segment_reduce(op, feats.data_ptr<float>(), p.sid.data_ptr<int>(), p.perm_ptr(),
                              p.offsets.data_ptr<int>(), flags, p.balance.data_ptr<int>(), int(p.balance.numel()), n,
                              int(c), m, out.data_ptr<float>(), arg_ptr, int32_t(arg_base), ws.data_ptr(),
                              size_t(ws.numel()), stream);
    check_status(st, "texb_segment_reduce (sequence)");
    results.emplace_back(out, arg);
    ++k;
  }
  return results;
}

// Autograd may hand over an expanded or strided gradient; the C ABI wants fp32 rows.
at::Tensor grad_rows(const Plan& p, const at::Tensor& g) {
  TORCH_CHECK(g.device().is_cuda(), "the gradient must be a CUDAtensor ");
  TORCH_CHECK(g.dim() == 2 && g.size(0) == p.num_segments, "the gradient must be [num_unq, channel]");
  TORCH_CHECK(g.device() == p.sid.device(), "the gradient and ScatterData live on different devices");
  return (g.scalar_type() == at::kFloat ? g : g.to(at::kFloat)).contiguous();
}

// mode: TEXB_OP_SUM g[unq_inv], TEXB_OP_MEAN (g / count)[unq_inv], TEXB_OP_MAX the gradient routed to arg.
at::Tensor broadcast_back(Plan& p, int mode, const at::Tensor& g_in, c10::optional<at::Tensor> arg) {
  const at::Tensor g = grad_rows(p, g_in);
  const int64_t n = p.num_total, c = g.size(1), m = p.num_segments;
  const c10::cuda::CUDAGuard guard(g.device());
  void* stream = stream_of(g);
  at::Tensor out = at::empty({n, c}, g.options());
  int st;
  if (mode == TEXB_OP_SUM) {
    st = texb_scatter_sum_backward(g.data_ptr<float>(), p.sid.data_ptr<int>(), p.perm_ptr(), out.data_ptr<float>(), n,
                                   int(c), m, stream);
  } else if (mode == TEXB_OP_MEAN) {
    st = texb_scatter_mean_backward(g.data_ptr<float>(), p.sid.data_ptr<int>(), p.perm_ptr(),
                                    p.offsets.data_ptr<int>(), out.data_ptr<float>(), n, int(c), m, stream);
  } else {
    TORCH_CHECK(mode == TEXB_OP_MAX, "unknown backward mode ", mode);
    TORCH_CHECK(arg.has_value(), "the max backward needs arg");
    TEXB_CHECK_INPUT((*arg));
    TEXB_CHECK_DTYPE((*arg), at::kInt);
    TORCH_CHECK(arg->sizes() == g.sizes(), "arg and the gradient differ in shape");
    st = texb_scatter_max_backward(g.data_ptr<float>(), arg->data_ptr<int>(), p.sid.data_ptr<int>(), p.perm_ptr(),
                                   out.data_ptr<float>(), n, int(c), m, stream);
  }
  check_status(st, "texb_scatter_*_backward");
  return out;
}

at::Tensor mean_max_backward(Plan& p, const at::Tensor& g_mean_in, const at::Tensor& g_max_in,
                             const at::Tensor& arg) {
  const at::Tensor g_mean = grad_rows(p, g_mean_in), g_max = grad_rows(p, g_max_in);
  TEXB_CHECK_INPUT(arg);
  TEXB_CHECK_DTYPE(arg, at::kInt);
  TORCH_CHECK(g_mean.sizes() == g_max.sizes() && arg.sizes() == g_mean.sizes(),
              "the two gradients and arg differ in shape");
  const int64_t n = p.num_total, c = g_mean.size(1), m = p.num_segments;
  const c10::cuda::CUDAGuard guard(g_mean.device());
  at::Tensor out = at::empty({n, c}, g_mean.options());
  check_status(texb_scatter_mean_max_backward(g_mean.data_ptr<float>(), g_max.data_ptr<float>(), arg.data_ptr<int>(),
                                              p.sid.data_ptr<int>(), p.perm_ptr(), p.offsets.data_ptr<int>(),
                                              out.data_ptr<float>(), n, int(c), m, stream_of(g_mean)),
               "texb_scatter_mean_max_backward");
  return out;
}

at::Tensor segment_rank(Plan& p) {
  const c10::cuda::CUDAGuard guard(p.sid.device());
  at::Tensor out = at::empty({p.num_total}, p.sid.options().dtype(at::kLong));
  check_status(texb_segment_rank(p.sid.data_ptr<int>(), p.perm_ptr(), p.offsets.data_ptr<int>(), p.num_total,
                                 p.num_segments, out.data_ptr<int64_t>(), stream_of(p.sid)),
               "texb_segment_rank");
  return out;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "scatter_ext: TorchEx's native scatter module on the B200 kernels (C ABI: texb_scatter.h)";
  m.def("sum", &scatter_sum_gpu, "scatter_sum (CUDA)");
  m.def("max", &scatter_max_gpu, "scatter_max (CUDA)");
  m.def("getPreSum", &get_pre_sum_gpu, "get preSum from unq_inv (CUDA)");

  py::class_<Plan>(m, "Plan")
      .def_readonly("sid", &Plan::sid)
      .def_readonly("offsets", &Plan::offsets)
      .def_readonly("balance", &Plan::balance)
      .def_readonly("num_total", &Plan::num_total)
      .def_readonly("num_segments", &Plan::num_segments)
      .def_readwrite("max_cnt", &Plan::max_cnt)
      .def_readwrite("has_empty", &Plan::has_empty)
      .def_readwrite("settled", &Plan::settled)
      .def_readwrite("no_split", &Plan::no_split)
      .def("scratch_buffers", [](const Plan& p) { return p.scratch_cache.size(); },
           "number of reduce workspaces the plan holds (one per channel count, operator kind and stream)");
  m.def("make_plan", &make_plan, py::arg("sid"), py::arg("perm"), py::arg("offsets"), py::arg("balance"),
        py::arg("num_segments"), py::arg("has_empty"), py::arg("max_cnt"), py::arg("settled"));
  m.def("build_plan", &build_plan, py::arg("ids"), py::arg("num_segments"), py::arg("balance_pieces"));
  m.def("reduce", &reduce, py::arg("plan"), py::arg("op"), py::arg("feats"), py::arg("arg_base") = 0,
        py::arg("out") = c10::nullopt, py::arg("arg") = c10::nullopt);
  m.def("reduce_sequence", &reduce_sequence, py::arg("plan"), py::arg("ops"), py::arg("feats"),
        py::arg("arg_base") = 0);
  m.def("reduce_pair", &reduce_pair, py::arg("plan"), py::arg("op"), py::arg("feats"), py::arg("arg_base") = 0,
        py::arg("out_sum") = c10::nullopt, py::arg("out_max") = c10::nullopt, py::arg("arg") = c10::nullopt);
  m.def("broadcast_back", &broadcast_back, py::arg("plan"), py::arg("mode"), py::arg("g"),
        py::arg("arg") = c10::nullopt);
  m.def("mean_max_backward", &mean_max_backward);
  m.def("segment_rank", &segment_rank);
  m.def("abi_version", &texb_version);
}
