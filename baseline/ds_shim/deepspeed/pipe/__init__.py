from ..runtime.pipe.module import PipelineModule, LayerSpec, TiedLayerSpec  # noqa: F401
