from .registry import build_model, detect_model_type, MODEL_REGISTRY  # noqa: F401
