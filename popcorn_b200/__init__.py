"""popcorn_b200: one CUDA (sm_100a) backend for popcorn's memory-bound transformer-layer ops.

    from popcorn_b200 import ops                 # rms_norm, add_rms_norm, rotary_embedding, swiglu, moe_*
    from popcorn_b200.kernels import rms_norm    # the same ops behind popcorn's call surface
    import popcorn_b200.plugin                   # plugin.register() attaches them to popcorn itself

Importing the package does not load the shared library; the first op call does,
and raises if libpopcorn_b200.so has not been built (python -m popcorn_b200.build).
"""

__version__ = "0.1.0"
