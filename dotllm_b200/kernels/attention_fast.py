"""Dispatch to the tensor-core attention kernels for the sizes they take."""


def run(q, q_stride, out, k_pool, v_pool, n_pages, token_seq, token_pos, block_table,
        n_heads, n_kv_heads, head_dim, scale, window, plan):
    """Run a tensor-core kernel into ``out`` and return True, or return False to let the
    generic kernel take the call."""
    return False
