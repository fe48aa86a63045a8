"""Host-side partition rules of expert-parallel decode (the device side is sl_ep_init /
sl_batch_step_argmax in the C ABI).  Experts are split into equal contiguous ranges; streams are
dealt to ranks in contiguous blocks so that rank r's rows sit at offset r*rows_per_rank of every
gathered buffer."""


def expert_range(rank, world, n_experts):
    if n_experts % world:
        raise ValueError("the expert count must divide evenly across ranks")
    per = n_experts // world
    return rank * per, (rank + 1) * per


def streams_of_rank(rank, world, n_streams):
    if n_streams % world:
        raise ValueError("the stream count must divide evenly across ranks (pad the batch)")
    per = n_streams // world
    return list(range(rank * per, (rank + 1) * per))


def owner_of_expert(expert, world, n_experts):
    return expert // (n_experts // world)


def pair_slices(rank, rows_per_rank, top_k):
    """[start, stop) of this rank's (row, k) pairs in the global pair numbering t*top_k + k."""
    return rank * rows_per_rank * top_k, (rank + 1) * rows_per_rank * top_k
