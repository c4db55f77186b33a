"""Names of the reference's extension layer (Transformer Engine adapter, spec providers) backed by this library's
own kernels, so that model code written against those names ports without edits."""
