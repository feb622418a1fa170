"""Tinker-compatible training/sampling service: REST API, sqlite request store, batching engine loop, backend adapter."""
