"""Exception types shared by the kernels' host wrappers and the runtime."""


class CollectiveTimeout(RuntimeError):
    """A collective (a device-side bounded wait or a c10d operation) did not complete in time."""


class CheckpointError(RuntimeError):
    """A checkpoint file could not be read back (missing, truncated or not a checkpoint)."""
