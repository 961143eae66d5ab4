"""Module paths of the reference's ``fms_acceleration_foak.kernels`` package, bound to the in-tree operators."""
