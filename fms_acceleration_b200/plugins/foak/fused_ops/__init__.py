"""Module paths of the reference's ``fms_acceleration_foak.fused_ops`` package, bound to the in-tree operators."""
