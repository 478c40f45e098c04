"""The architectures this package brings. Importing this module registers them; another
architecture is added the same way from anywhere: a typed config reader, a builder of a
:class:`~hi_b200.parts.spec.ModelSpec` and a tensor-name normaliser, handed to
:func:`~hi_b200.config.registry.register_architecture` under its ``architectures`` /
``model_type`` names (the reference routes ``llama4`` / ``llama4_text`` to its Llama 4 model:
crates/hi-mlx/src/config.rs:620-637, crates/hi-mlx/src/models.rs:373-375)."""
from .config import bezasun as _bezasun
from .config import fidatar as _fidatar
from .config import surinex as _surinex
from .config import vinurax as _vinurax
from .config.llama4 import Llama4TextConfig
from .config.registry import Architecture, register_architecture
from .parts.bezasun import build_bezasun_spec, normalize_bezasun_tensor_name
from .parts.fidatar import build_fidatar_spec, normalize_fidatar_tensor_name
from .parts.llama4 import build_llama4_spec, derive_llama4_tensors, normalize_llama4_tensor_name
from .parts.surinex import build_surinex_spec, normalize_surinex_tensor_name
from .parts.vinurax import build_vinurax_spec, normalize_vinurax_tensor_name

register_architecture(
    ["Llama4ForConditionalGeneration", "Llama4ForCausalLM", "llama4", "llama4_text"],
    Architecture(name="llama4_text", parse_config=Llama4TextConfig.from_json, build_spec=build_llama4_spec,
                 normalize_tensor_name=normalize_llama4_tensor_name, derive_tensors=derive_llama4_tensors))

register_architecture(
    ["Vinurax", "vinurax"],
    Architecture(name="vinurax", parse_config=_vinurax.VinuraxConfig.from_json, build_spec=build_vinurax_spec,
                 normalize_tensor_name=normalize_vinurax_tensor_name, sizes_from_tensors=_vinurax.sizes_from_tensors))

register_architecture(
    ["Fidatar", "fidatar"],
    Architecture(name="fidatar", parse_config=_fidatar.FidatarConfig.from_json, build_spec=build_fidatar_spec,
                 normalize_tensor_name=normalize_fidatar_tensor_name))

register_architecture(
    ["Surinex", "surinex"],
    Architecture(name="surinex", parse_config=_surinex.SurinexConfig.from_json, build_spec=build_surinex_spec,
                 normalize_tensor_name=normalize_surinex_tensor_name, sizes_from_tensors=_surinex.sizes_from_tensors))

register_architecture(
    ["Bezasun", "bezasun"],
    Architecture(name="bezasun", parse_config=_bezasun.BezasunConfig.from_json, build_spec=build_bezasun_spec,
                 normalize_tensor_name=normalize_bezasun_tensor_name))
