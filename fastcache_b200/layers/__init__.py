"""Model building blocks (linear family, attention, embeddings, norms, rotary, activation, sampler)."""
