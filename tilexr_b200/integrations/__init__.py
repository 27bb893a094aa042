"""Framework integrations: MoonEP-compatible buffer, vLLM communicator patch."""
