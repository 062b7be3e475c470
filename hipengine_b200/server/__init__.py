"""OpenAI-compatible server package."""
