"""Dispatch to the weight-streaming product for steps of a few rows (decode)."""


def maybe_run(x, w, out_dtype):
    """y = x W^T by the skinny kernel when it takes the sizes, else None."""
    return None
