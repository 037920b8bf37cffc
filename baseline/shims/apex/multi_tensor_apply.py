"""`apex.multi_tensor_apply` without `amp_C`: the applier exists and says it is unavailable."""


class MultiTensorApply:
    available = False
    warned = False

    def __init__(self, chunk_size):
        self.chunk_size = chunk_size

    def __call__(self, op, noop_flag_buffer, tensor_lists, *args):
        raise RuntimeError("apex multi_tensor_applier requires cuda extensions (amp_C)")


multi_tensor_applier = MultiTensorApply(2048 * 32)
