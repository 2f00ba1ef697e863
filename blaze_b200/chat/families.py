"""Family dispatch for the built-in prompt encoders: which encoder a checkpoint gets, from its name and ``config.json``.
Reference: ``crates/blaze-chat/src/render/selection.rs`` (``select_chat_formatter``)."""
from __future__ import annotations

from typing import Any, Dict, Optional, Tuple


def encoder_of(model: str, config: Optional[Dict[str, Any]] = None) -> Optional[str]:
    """Name of the built-in request encoder for a checkpoint, or None when only the template renderer applies."""
    config = config or {}
    mt = str(config.get("model_type") or "").lower()
    archs = " ".join(config.get("architectures") or []).lower()
    name = (model or "").lower()
    if mt == "deepseek_v41" or "deepseekv41" in archs or "deepseek-v4.1" in name:
        return "deepseek_v41"
    if mt == "deepseek_v4" or "deepseekv4" in archs or "deepseek-v4" in name:
        return "deepseek_v4"
    if mt == "kimi_k3" or "kimik3" in archs or "kimi-k3" in name:
        return "kimi_k3"
    return None


def render_request(model: str, config: Dict[str, Any], request: Dict[str, Any],
                   defaults: Optional[Dict[str, Any]] = None, chat_template: Optional[str] = None) -> Tuple[str, str]:
    """``(prompt, continuation prefix)`` of a chat request through the checkpoint's built-in encoder, or through its
    ``chat_template`` with the family's request preparation."""
    enc = encoder_of(model, config)
    if enc is None and chat_template:
        from . import templated
        fam = "glm53" if templated.is_glm53(chat_template) else "qwen38" if templated.is_qwen38(chat_template) else None
        if fam is not None:
            from .template import ChatFormatter
            return templated.render_request(ChatFormatter(chat_template), request, defaults, fam)
    if enc in ("deepseek_v4", "deepseek_v41"):
        from . import deepseek
        return deepseek.render_request(request, defaults, v41=enc == "deepseek_v41",
                                       profile=str(config.get("dsv4_reasoning_effort_profile") or "preview"))
    if enc == "kimi_k3":
        from . import kimi
        return kimi.render_request(request, defaults)
    raise ValueError(f"no built-in request encoder for {model!r}")
