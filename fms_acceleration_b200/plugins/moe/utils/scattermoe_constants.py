"""Names and per-architecture conversion specs of the ScatterMoE module swap (same values as
fms_acceleration_moe/utils/scattermoe_constants.py:19-108 of the reference)."""
from typing import List

PARAM_NAME_ROUTER_SCATTERMOE = "router"
PARAM_NAME_WEIGHT_SCATTERMOE = ["w1", "w2", "w3"]  # w1: activated (gate) proj, w3: multiplicative (up) proj, w2: down proj
FILE_SAFETENSOR_INDEX = "model.safetensors.index.json"
KEY_REPLICATE = "replicate"
KEY_EXPERT_PARALLEL = "expert_parallel"
DIM_EXPERT = 0
KEY_SCATTERMOE_ROUTER = PARAM_NAME_ROUTER_SCATTERMOE + ".weight"
SCATTERMOE_SPEC_HAS_GATE = "Gated"

# architecture -> (MoE block class name, router attribute, expert attribute(s) in w1|w2|w3 order, gating, whether
# the checkpoint stores one linear per expert)
SCATTERMOE_CONVERSION_SPEC = {
    "MixtralForCausalLM": ("MixtralSparseMoeBlock", "gate", "experts", SCATTERMOE_SPEC_HAS_GATE, True),
    "GraniteMoeForCausalLM": ("GraniteMoeMoE", "router", "input_linear|output_linear|input_linear",
                              SCATTERMOE_SPEC_HAS_GATE, False),
    "GraniteMoeSharedForCausalLM": ("GraniteMoeSharedMoE", "router", "input_linear|output_linear|input_linear",
                                    SCATTERMOE_SPEC_HAS_GATE, False),
    "GraniteMoeHybridForCausalLM": ("GraniteMoeHybridMoE", "router", "input_linear|output_linear|input_linear",
                                    SCATTERMOE_SPEC_HAS_GATE, False),
}


def get_scattermoe_conv_spec_from_archs(architectures: List[str]):
    for archs, spec in SCATTERMOE_CONVERSION_SPEC.items():
        if any(a in archs.split(",") for a in architectures):
            return spec
    raise ValueError(
        f"In order to configure ScatterMoe for archs '{architectures}' "
        "the conversion spect must be updated in scattermoe_constants.py"
    )
