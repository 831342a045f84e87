"""svoo_b200: SVOO's online sparse-attention path on hand-written sm_100a CUDA kernels.

Sub-modules (imported on demand; everything except `synth`, `sparsity` and `build`
loads libsvoo_b200.so and raises if it is missing -- there is no fallback):

  co_clustering  co_cluster_tokens, identify_dynamic_map, dynamic_block_sparse_fwd_*, batch_kmeans_Euclid
  permute        permute_tensor_by_labels(_triton), apply_inverse_permutation(_triton)
  sparsity       SparsityLookup and the per-head density clipping
  layer          sparse_attention_layer: the whole path as one kernel sequence
  processor      WanAttn_SAPAttn_Processor, Hunyuan_SAPAttn_Processor2_0
  parallel       head-sharded (Ulysses) execution: peer-store re-shard, head partition, host-shard pipeline
  wan_dit        a plain-torch DiT with the Wan block structure around the processor (in-situ runs)
  ops            one torch wrapper per C-ABI entry point
  synth          seeded synthetic workloads
  build          nvcc build of the shared library
"""
__version__ = "0.1.0"
