"""Serving-engine hooks: per-layer TurboQuant state with boundary-layer gating, and a vLLM attention backend."""
