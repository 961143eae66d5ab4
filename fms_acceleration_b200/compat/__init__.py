"""Stand-ins for the parts of ``accelerate`` / ``peft`` / ``transformers.TrainingArguments`` that the framework
touches, for machines where those packages are not installed."""
from .accelerator import Accelerator, AcceleratorState, FSDPPluginShim  # noqa: F401
from ..nn.lora import LoraConfig, LoraLinear, PeftModelShim, get_peft_model  # noqa: F401
from ..trainer import TrainArgs as TrainingArguments  # noqa: F401
