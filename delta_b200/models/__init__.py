"""Model specifications and the generic model that runs them."""
from ..config.model_config import YiConfig
from ..config.registry import register_architecture
from .model import Model
from .spec import LayerSpec, ModelSpec, RunEntry
from .yi import yi_spec
from .roletar import roletar_spec
from .pibalorn import pibalorn_spec
from .mufalix import mufalix_spec
from .mevulix import mevulix_spec
from ..config.roletar_config import RoletarConfig
from ..config.pibalorn_config import PibalornConfig
from ..config.mufalix_config import MufalixConfig
from ..config.mevulix_config import MevulixConfig, sizes_from_shapes as _mevulix_sizes
from ..parts import (decay_attention, experts, gated_recurrence, latent_attention, matrix_memory, residual,  # noqa: F401
                     row_attention, selective_scan, side_by_side, streams)  # (register their parts)

for _name in ("LlamaForCausalLM", "YiForCausalLM"):
    register_architecture(_name, YiConfig.from_dict, yi_spec)
register_architecture("Roletar", RoletarConfig.from_dict, roletar_spec)
register_architecture("Pibalorn", PibalornConfig.from_dict, pibalorn_spec)
register_architecture("Mufalix", MufalixConfig.from_dict, mufalix_spec)
register_architecture("Mevulix", MevulixConfig.from_dict, mevulix_spec, sizes_from_shapes=_mevulix_sizes)
