"""Small helpers that are no part of the model: tracing."""
