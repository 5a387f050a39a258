from .attention import attention, TAU, EPS, CLAMP

__all__ = ["attention", "TAU", "EPS", "CLAMP"]
