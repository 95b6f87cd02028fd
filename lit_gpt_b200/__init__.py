"""b200gpt: B200-native (sm_100a) implementation of lit-gpt's quantized decode/prefill hot path.

Public surface mirrors the reference package (``from lit_gpt import GPT, Config``) plus the quantization plugin that
replaces ``lightning.fabric.plugins.BitsandbytesPrecision``.
"""
from lit_gpt_b200.config import Config, FizadraConfig, LefalixConfig, NulezenConfig, PomipelConfig, load_config, model_class
from lit_gpt_b200.fizadra import Fizadra
from lit_gpt_b200.lefalix import Lefalix
from lit_gpt_b200.nulezen import Nulezen
from lit_gpt_b200.model import GPT
from lit_gpt_b200.pomipel import Pomipel
from lit_gpt_b200.quant import QLinear, QuantPrecision
from lit_gpt_b200.rmsnorm import RMSNorm

__all__ = ["GPT", "Config", "Fizadra", "FizadraConfig", "Lefalix", "LefalixConfig", "Nulezen", "NulezenConfig", "Pomipel", "PomipelConfig", "QLinear", "QuantPrecision", "RMSNorm", "load_config", "model_class"]
__version__ = "0.1.0"
