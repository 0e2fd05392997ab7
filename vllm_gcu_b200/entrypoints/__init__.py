"""Serving entry points: OpenAI-compatible HTTP server and offline helpers."""
