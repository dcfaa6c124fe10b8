"""CPU oracle for the adaptive hybrid quantization path (test infrastructure only).

Nothing in ``atlasinfer_b200`` imports this package.  See ``atlas_oracle.c`` for
the arithmetic and ``atlas_oracle.py`` for the ctypes wrapper.
"""
