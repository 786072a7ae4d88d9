"""CUDA kernels for the TurboQuant hot paths (sm_100a), behind the reference's module names.

Modules: packed_compress (compress_k, compress_k_permuted, compress_v and the
pack/unpack helpers), packed_attention (packed_attention, attention_unpacked_ref),
sparse_v (paged GQA decode with the Sparse-V rule), paged (the paged-cache
pair compress_and_scatter / paged_decode_attention), paged_layout (page format).
As in the reference, nothing is re-exported from the package itself.
"""
