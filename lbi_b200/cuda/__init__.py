"""Python entry points of the kernels under the module paths of the reference's ``cuda`` package
(cuda/interface, cuda/transformer, cuda/mamba3).  The kernels themselves live in ``csrc/`` and are built into one
extension; ``ops`` is the dispatch layer these functions call."""
