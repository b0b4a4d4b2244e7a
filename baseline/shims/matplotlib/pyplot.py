"""See the package docstring: an import stand-in, no drawing."""


def _unavailable(*_a, **_k):
    raise RuntimeError("matplotlib is not installed; schedule drawing is unavailable")


subplots = savefig = figure = show = close = _unavailable
