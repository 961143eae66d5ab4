"""Import paths of the reference's ``gptqmodel.nn_modules`` package, bound to the in-tree layer and kernels."""
