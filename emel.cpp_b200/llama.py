"""Decoder-session bindings (include/emelb_llama.h); filled in with the session API."""
