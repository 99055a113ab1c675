"""Small helpers kept for API parity with the reference package."""


def tune_cpu(*_args, **_kwargs):
    """The reference pins PyTorch's CPU threads to an M1 Pro's fast cores; on a B200 host there is nothing to pin.
    Returns None and changes nothing."""
    return None
