// One decode step of the DSA block for callers whose per-step tensors live in pinned HOST memory:
// copies in, both operators, copies out, one call.  The copies overlap the kernels on a second
// stream so that only the indexer's inputs (in) and the attention's output (out) are exposed:
//
//   main : H2D [q_index | weights | seq_lens | block_table] -> indexer -> (wait q) -> attention
//          -> D2H [output | lse] -> synchronise
//   side : (after the first copy) H2D [q_nope | q_pe]  ...  (after the indexer) D2H indices
//
// The reference's callers pass CUDA tensors (kbench/flashinfer.py:109-120); this entry is what a
// serving loop that builds its queries on the host calls instead of nine copies and two launches.
#include "common.cuh"

extern "C" int dsa_decode_step_host(const dsa_host_step_args* a) {
  if (a == nullptr) return DSA_ERR_NULL_POINTER;
  if (!a->host_in || !a->dev_in || !a->host_out || !a->dev_out || !a->ev_first_copy ||
      !a->ev_q_ready || !a->ev_indices_ready)
    return DSA_ERR_NULL_POINTER;
  if (a->batch <= 0 || a->in_indexer_bytes == 0 || a->in_attention_bytes == 0 ||
      a->out_attention_bytes == 0 || a->out_indices_bytes == 0)
    return DSA_ERR_BAD_SHAPE;
  cudaStream_t main_s = static_cast<cudaStream_t>(a->stream);
  cudaStream_t side_s = static_cast<cudaStream_t>(a->side_stream);
  cudaEvent_t ev_a = static_cast<cudaEvent_t>(a->ev_first_copy);
  cudaEvent_t ev_q = static_cast<cudaEvent_t>(a->ev_q_ready);
  cudaEvent_t ev_i = static_cast<cudaEvent_t>(a->ev_indices_ready);
  const char* hin = static_cast<const char*>(a->host_in);
  char* din = static_cast<char*>(a->dev_in);
  char* hout = static_cast<char*>(a->host_out);
  const char* dout = static_cast<const char*>(a->dev_out);
  cudaError_t e;
#define DSA_TRY(call) \
  if ((e = (call)) != cudaSuccess) return static_cast<int>(e)

  // indexer inputs first, alone on the link; the indexer follows at once
  DSA_TRY(cudaMemcpyAsync(din, hin, a->in_indexer_bytes, cudaMemcpyHostToDevice, main_s));
  DSA_TRY(cudaEventRecord(ev_a, main_s));
  int rc = dsa_indexer_topk(a->q_index_fp8, a->k_index_cache, a->weights, a->seq_lens,
                            a->block_table, a->block_table_stride, a->topk_indices, DSA_TOPK,
                            a->batch, a->num_pages, a->max_pages, a->indexer_workspace,
                            a->indexer_workspace_bytes, a->status_dev, a->stream);
  if (rc != DSA_OK) return rc;
  DSA_TRY(cudaEventRecord(ev_i, main_s));
  // the attention's queries travel under the indexer
  DSA_TRY(cudaStreamWaitEvent(side_s, ev_a, 0));
  DSA_TRY(cudaMemcpyAsync(din + a->in_indexer_bytes, hin + a->in_indexer_bytes,
                          a->in_attention_bytes, cudaMemcpyHostToDevice, side_s));
  DSA_TRY(cudaEventRecord(ev_q, side_s));
  DSA_TRY(cudaStreamWaitEvent(main_s, ev_q, 0));
  rc = dsa_sparse_attn(a->q_nope, a->q_pe, a->ckv_cache, a->kpe_cache, a->topk_indices, DSA_TOPK,
                       a->sm_scale, a->output, a->lse, a->batch, DSA_ATTN_HEADS, DSA_TOPK,
                       a->num_slots, a->attention_workspace, a->attention_workspace_bytes,
                       a->status_dev, a->stream);
  if (rc != DSA_OK) return rc;
  // the indices travel back under the attention, output and LSE after it
  DSA_TRY(cudaStreamWaitEvent(side_s, ev_i, 0));
  DSA_TRY(cudaMemcpyAsync(hout + a->out_attention_bytes, dout + a->out_attention_bytes,
                          a->out_indices_bytes, cudaMemcpyDeviceToHost, side_s));
  DSA_TRY(cudaMemcpyAsync(hout, dout, a->out_attention_bytes, cudaMemcpyDeviceToHost, main_s));
  DSA_TRY(cudaStreamSynchronize(side_s));
  DSA_TRY(cudaStreamSynchronize(main_s));
#undef DSA_TRY
  return DSA_OK;
}
