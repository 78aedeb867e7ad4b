"""HTTP serving layer: OpenAI / Anthropic / llama-server compatible API over the engine."""
