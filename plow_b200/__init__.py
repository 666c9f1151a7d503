"""plow_b200 — a Blackwell-native (sm_100a) ahead-of-time LLM inference compiler and serving runtime.

``plowc`` lowers a checkpoint's ``config.json`` into a packet (tensor table + one pre-planned
program per prefill bucket / decode rung); ``plowrt`` loads packet + safetensors weights, runs a
continuous-batching scheduler over a paged KV cache and serves an OpenAI-compatible API.
"""
__version__ = "0.1.0"
