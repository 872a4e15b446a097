"""Model registry: config.json names the architecture, the registry maps it to the loader that builds the model
object the runners and the engine drive.  REF mistralrs-core/src/pipeline/loaders (`NormalLoaderType` chosen from
the `architectures` entry of config.json)."""
import json
import os

_LOADERS = {}


def register(architecture, loader):
    """loader(model_dir, device, dtype, **options) -> model object."""
    _LOADERS[architecture] = loader


def architecture_of(cj: dict) -> str:
    if "architecture" in cj:
        return str(cj["architecture"])
    if cj.get("architectures"):
        return str(cj["architectures"][0])
    if "model_type" in cj:
        return str(cj["model_type"])
    raise ValueError("config.json names no architecture")


def registered():
    return sorted(_LOADERS)


def load_model(model_dir, device, dtype, **options):
    with open(os.path.join(model_dir, "config.json")) as f:
        arch = architecture_of(json.load(f))
    if arch not in _LOADERS:
        raise NotImplementedError(f"architecture {arch!r} is not registered (known: {', '.join(registered())})")
    return _LOADERS[arch](model_dir, device, dtype, **options)


def _load_nisasun(model_dir, device, dtype, **options):
    from .nisasun import NisasunModel
    return NisasunModel.from_dir(model_dir, device, dtype, **options)


def _load_kilizen(model_dir, device, dtype, **options):
    from .kilizen import KilizenModel
    return KilizenModel.from_dir(model_dir, device, dtype, **options)


def _load_fosulix(model_dir, device, dtype, **options):
    from .fosulix import FosulixModel
    return FosulixModel.from_dir(model_dir, device, dtype, **options)


def _load_kibotar(model_dir, device, dtype, **options):
    from .kibotar import KibotarModel
    return KibotarModel.from_dir(model_dir, device, dtype, **options)


def _load_llama(model_dir, device, dtype, **options):
    """Llama-family UQFF folder (config.json + *.uqff shards + residual.safetensors) -> `model.LlamaWeights`, the object
    `model.LlamaRunner` / `model.LlamaPrefill` drive."""
    from . import model, uqff_file
    shards = sorted(os.path.join(model_dir, f) for f in os.listdir(model_dir) if f.endswith(".uqff"))
    if not shards:
        raise FileNotFoundError(f"{model_dir} holds no .uqff shard (llama-family checkpoints load from UQFF or GGUF)")
    with open(os.path.join(model_dir, "config.json")) as f:
        cj = json.load(f)
    residual = os.path.join(model_dir, "residual.safetensors")
    ar = uqff_file.UqffArchive(shards, residual=residual if os.path.exists(residual) else None, config=cj)
    return model.LlamaWeights.from_uqff(ar, device, dtype, **options)


register("Nisasun", _load_nisasun)
register("Kilizen", _load_kilizen)
register("Fosulix", _load_fosulix)
register("Kibotar", _load_kibotar)
for _name in ("LlamaForCausalLM", "MistralForCausalLM", "llama", "mistral"):
    register(_name, _load_llama)
