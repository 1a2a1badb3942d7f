// Thin PyTorch extension over the C ABI: registers `torch.ops.asymgemm_b200.m_grouped_gemm_nt`, the one launch every
// operator of the Python API funnels into. It plays the part of the reference's pybind layer (csrc/apis/gemm.hpp:1034-1115
// binds the operators, csrc/jit/kernel_runtime.hpp:99-119 launches on torch's current stream): take tensors, fill the
// plain descriptor, launch on the current CUDA stream of a's device, turn a failure into c10::Error (RuntimeError in
// Python). No arithmetic happens here and nothing is allocated; the library below it has no torch dependency.
#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include "../../include/asymgemm_b200.h"

namespace {

using OptTensor = c10::optional<at::Tensor>;

void* ptr_of(const OptTensor& t) { return t.has_value() && t->defined() ? t->data_ptr() : nullptr; }

void check_index_tensor(const OptTensor& t, const char* name, const at::Tensor& a) {
  if (!t.has_value() || !t->defined()) return;
  TORCH_CHECK(t->is_cuda() && t->device() == a.device(), name, " must live on a's device");
  TORCH_CHECK(t->scalar_type() == at::kInt && t->is_contiguous(), name, " must be a contiguous int32 tensor");
}

// kind: 0 bf16, 1 fp8 (fp32 scales), 2 int8, 3 nvfp4, 4 fp8 with blocked UE8M0 scales. layout: 0 contiguous, 1 masked.
void m_grouped_gemm_nt(int64_t kind, int64_t layout, const at::Tensor& a, const OptTensor& sfa, const at::Tensor& b,
                       const OptTensor& sfb, at::Tensor& d, const OptTensor& offsets, const OptTensor& experts,
                       int64_t max_segments, const OptTensor& masked_m, int64_t m, int64_t n, int64_t k, int64_t num_groups,
                       const OptTensor& scratch, const at::Tensor& status, int64_t timeout_ms, const OptTensor& raw_dump,
                       double alpha, int64_t tile_config, int64_t no_split, const OptTensor& stage, int64_t stage_chunk_bytes,
                       int64_t num_sms, int64_t epilogue, const OptTensor& scatter_meta, const OptTensor& scatter_bases) {
  TORCH_CHECK(a.is_cuda(), "a must be a CUDA tensor");
  TORCH_CHECK(b.is_cuda() || b.is_pinned(), "b must be a CUDA tensor or pinned host memory (b.is_cuda() or b.is_pinned())");
  TORCH_CHECK(d.is_cuda() || d.is_pinned(), "d must be a CUDA tensor or pinned host memory");
  TORCH_CHECK(a.is_contiguous() && b.is_contiguous() && d.is_contiguous(), "a, b and d must be contiguous");
  TORCH_CHECK(d.scalar_type() == at::kBFloat16 || d.scalar_type() == at::kFloat, "d must be bfloat16 or float32");
  TORCH_CHECK(status.is_cuda() && status.device() == a.device() && status.scalar_type() == at::kInt && status.numel() >= 1,
              "status must be an int32 tensor on a's device");
  check_index_tensor(offsets, "offsets", a);
  check_index_tensor(experts, "experts", a);
  check_index_tensor(masked_m, "masked_m", a);
  if (raw_dump.has_value() && raw_dump->defined())
    TORCH_CHECK(raw_dump->is_cuda() && raw_dump->scalar_type() == at::kInt && raw_dump->is_contiguous(),
                "raw_dump must be a contiguous int32 CUDA tensor");

  ag_gemm_desc_t desc{};
  desc.layout = static_cast<int32_t>(layout);
  desc.d_dtype = d.scalar_type() == at::kFloat ? AG_D_FP32 : AG_D_BF16;
  desc.a = a.data_ptr();
  desc.sfa = ptr_of(sfa);
  desc.b = b.data_ptr();
  desc.sfb = ptr_of(sfb);
  desc.d = d.data_ptr();
  desc.offsets = static_cast<const int32_t*>(ptr_of(offsets));
  desc.experts = static_cast<const int32_t*>(ptr_of(experts));
  desc.max_segments = static_cast<int32_t>(max_segments);
  desc.masked_m = static_cast<const int32_t*>(ptr_of(masked_m));
  desc.m = m;
  desc.n = n;
  desc.k = k;
  desc.num_groups = static_cast<int32_t>(num_groups);
  if (scratch.has_value() && scratch->defined()) {
    desc.scratch = scratch->data_ptr();
    desc.scratch_bytes = static_cast<uint64_t>(scratch->numel()) * scratch->element_size();
  }
  desc.status = static_cast<int32_t*>(status.data_ptr());
  desc.epilogue = static_cast<int32_t>(epilogue);
  const bool has_meta = scatter_meta.has_value() && scatter_meta->defined();
  const bool has_bases = scatter_bases.has_value() && scatter_bases->defined();
  TORCH_CHECK(has_meta == has_bases, "scatter_meta and scatter_bases go together");
  if (has_meta) {
    TORCH_CHECK(scatter_meta->is_cuda() && scatter_meta->device() == a.device() && scatter_meta->scalar_type() == at::kLong &&
                    scatter_meta->is_contiguous() && scatter_meta->numel() >= m,
                "scatter_meta must be a contiguous int64 tensor on a's device with one entry per row of a");
    TORCH_CHECK(scatter_bases->is_cuda() && scatter_bases->device() == a.device() && scatter_bases->scalar_type() == at::kLong &&
                    scatter_bases->is_contiguous() && scatter_bases->numel() >= 1,
                "scatter_bases must be a contiguous int64 tensor of buffer addresses on a's device");
    desc.scatter_meta = static_cast<const int64_t*>(scatter_meta->data_ptr());
    desc.scatter_bases = static_cast<const int64_t*>(scatter_bases->data_ptr());
  }
  desc.num_sms = static_cast<int32_t>(num_sms > 0 ? num_sms : 0);   // 0: every SM, or the process-wide cap
  desc.timeout_ms = static_cast<uint32_t>(timeout_ms);
  desc.raw_dump = static_cast<int32_t*>(ptr_of(raw_dump));
  desc.alpha = static_cast<float>(alpha);
  desc.tile_config = static_cast<int32_t>(tile_config);
  desc.no_split = static_cast<int32_t>(no_split);
  if (stage.has_value() && stage->defined()) {
    TORCH_CHECK(stage->is_cuda() && stage->device() == a.device(), "stage must live on a's device");
    desc.stage = stage->data_ptr();
    desc.stage_bytes = static_cast<uint64_t>(stage->numel()) * stage->element_size();
    desc.stage_chunk_bytes = static_cast<uint64_t>(stage_chunk_bytes > 0 ? stage_chunk_bytes : 0);
  }

  int rc = AG_E_INVALID;
  {
    // device guard and launch in a scope of their own: a failure is raised after the guard has been released
    const c10::cuda::CUDAGuard guard(a.device());
    desc.stream = c10::cuda::getCurrentCUDAStream(a.device().index()).stream();
    switch (kind) {
      case 0: rc = ag_m_grouped_bf16_gemm_nt(&desc); break;
      case 1: rc = ag_m_grouped_fp8_gemm_nt(&desc); break;
      case 2: rc = ag_m_grouped_int8_gemm_nt(&desc); break;
      case 3: rc = ag_m_grouped_fp4_gemm_nt(&desc); break;
      case 4: rc = ag_m_grouped_fp8_ue8m0_gemm_nt(&desc); break;
      default: rc = AG_E_UNSUPPORTED; break;
    }
  }
  TORCH_CHECK(rc != AG_E_UNSUPPORTED || (kind >= 0 && kind <= 4), "asymgemm_b200: unknown kind ", kind);
  TORCH_CHECK(rc == AG_OK, "asymgemm_b200: ", ag_last_error(), " (code ", rc, ")");
}

}  // namespace

TORCH_LIBRARY(asymgemm_b200, m) {
  m.def(
      "m_grouped_gemm_nt(int kind, int layout, Tensor a, Tensor? sfa, Tensor b, Tensor? sfb, Tensor(a!) d, Tensor? offsets, "
      "Tensor? experts, int max_segments, Tensor? masked_m, int m, int n, int k, int num_groups, Tensor? scratch, "
      "Tensor status, int timeout_ms, Tensor? raw_dump, float alpha, int tile_config, int no_split, Tensor? stage, int stage_chunk_bytes, "
      "int num_sms, int epilogue, Tensor? scatter_meta, Tensor? scatter_bases) -> ()");
}

TORCH_LIBRARY_IMPL(asymgemm_b200, CUDA, m) { m.impl("m_grouped_gemm_nt", &m_grouped_gemm_nt); }
