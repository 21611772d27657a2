"""mtb200: minitensor's dense-contraction path on B200 (sm_100a).

The package is a host-side mirror of the slice of minitensor's Python surface
that sits on that path (``Tensor.matmul`` / ``bmm``, ``nn.DenseLayer``,
``nn.Conv2d``, ``nn.cross_entropy``, ``optim.Adam``) over the C ABI of
``libmtb200.so``.  There is no CPU fallback: without the built library and a
B200 the operators raise.
"""
__version__ = "0.1.0"
