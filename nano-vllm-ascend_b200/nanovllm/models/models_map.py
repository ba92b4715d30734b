"""Which decoder class serves which HF ``architectures`` entry.

The dense families of the hot-path scope and the Qwen3-MoE stack are registered;
the reference's registry (models/models_map.py) also lists its MiniCPM and vision-language stacks,
which this build deliberately leaves out. Zegopel (a hybrid of softmax attention, lightning attention and
Mamba-2 layers) and Nirelix (retention, gated delta rule and latent attention on a residual kept in several
streams) and Fitevik (HGRN2 recurrences and attention with mixed heads, a distance bias and a sink, on a residual
with the norm on each sublayer's output) and Nurilorn (gated attention with capped scores, a sink, rotary positions
stretched band by band and values blended across layers, on a residual with scaled branches and grouped norms) are
additions; their config.json names them with an ``"architecture"`` string (config.NativeConfig). Qwen2 checkpoints are served by the Qwen3 class, as in the reference:
the config's ``attention_bias`` decides between QKV bias (Qwen2) and QK-norm (Qwen3).
"""
from __future__ import annotations

from .llama import LlamaForCausalLM
from .qwen3 import Qwen3ForCausalLM
from .qwen3_moe import Qwen3MoeForCausalLM
from .fitevik import FitevikForCausalLM
from .nirelix import NirelixForCausalLM
from .nurilorn import NurilornForCausalLM
from .zegopel import ZegopelForCausalLM

model_dict: dict[str, type] = {}


def register(architecture: str, cls: type) -> None:
    model_dict[architecture] = cls


for _arch, _cls in (("Qwen3ForCausalLM", Qwen3ForCausalLM),
                    ("Qwen2ForCausalLM", Qwen3ForCausalLM),
                    ("Qwen3MoeForCausalLM", Qwen3MoeForCausalLM),
                    ("LlamaForCausalLM", LlamaForCausalLM),
                    ("Zegopel", ZegopelForCausalLM),
                    ("Nirelix", NirelixForCausalLM),
                    ("Fitevik", FitevikForCausalLM),
                    ("Nurilorn", NurilornForCausalLM)):
    register(_arch, _cls)
