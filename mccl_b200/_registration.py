"""Glue between ``torch.distributed``'s backend registry and the native creator."""
from __future__ import annotations


def make_create_fn(native_create):
    """Adapts the native creator to c10d's extended registration API.

    ``init_process_group(..., pg_options=MCCLOptions(...))`` is honoured: the
    options object is passed to the process group as is; otherwise options are
    read from the ``MCCL_*`` environment.
    """

    def _create(dist_backend_opts, pg_options):
        from . import _C

        store = dist_backend_opts.store
        rank = dist_backend_opts.group_rank
        size = dist_backend_opts.group_size
        if isinstance(pg_options, _C.MCCLOptions):
            return _C.ProcessGroupMCCL(store, rank, size, pg_options)
        return native_create(store, rank, size, dist_backend_opts.timeout)

    return _create
