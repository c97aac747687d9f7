"""Terminal client: REPL over the OpenAI-compatible SSE endpoint and the agent-workload harness."""
