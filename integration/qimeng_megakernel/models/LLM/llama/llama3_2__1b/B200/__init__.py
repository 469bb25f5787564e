"""B200 implementation of this model (decode schedule packages; the kernels live in libqmk_b200.so)."""
