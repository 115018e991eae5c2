"""Model descriptions (one module per architecture) and the generic model
that is built from a description."""
