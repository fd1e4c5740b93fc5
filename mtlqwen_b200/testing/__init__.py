"""Helpers for tests and benchmarks: seeded synthetic weights / GGUF files and a decoder of the activation-image
layout. Nothing in the library proper imports this subpackage."""
