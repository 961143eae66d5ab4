"""Row permutations between the token layout and the expert-bin layout, and the differentiable all-to-all, under the
module names the reference vendors from MegaBlocks (scattermoe_utils/megablocks/)."""
from .autograd import all_to_all, gather, scatter  # noqa: F401,E402
