"""``multi_tensor_applier`` with Transformer Engine's calling convention."""

CHUNK_SIZE = 2048 * 32


def multi_tensor_applier(op, noop_flag_buffer, tensor_lists, *args):
    return op(CHUNK_SIZE, noop_flag_buffer, tensor_lists, *args)
