"""Sizes that the kernels take, as plain numbers: a configuration or a part can refuse what lies outside when a model
is put together, before a weight is read, instead of at its first step.  (The kernels check again at every launch.)"""

HEAD_DIM_STEP = 16          # attention takes head sizes that are multiples of this ...
MAX_HEAD_DIM = 256          # ... up to this (csrc/attention.cu: QWB_MAX_HEAD_DIM)


def head_dim_refusal(head_dim: int) -> str | None:
    """None if the attention kernels take this head size, else why not."""
    if head_dim <= 0 or head_dim % HEAD_DIM_STEP or head_dim > MAX_HEAD_DIM:
        return (f"the attention kernels take head sizes that are multiples of {HEAD_DIM_STEP} from {HEAD_DIM_STEP} to "
                f"{MAX_HEAD_DIM}, not {head_dim}")
    return None
