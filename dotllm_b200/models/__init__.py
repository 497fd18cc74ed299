"""Architectures (builders from a typed configuration to a model description) and the
generic decoder that runs any description."""
