"""Model-level mirrors of xax/arch (attention block and decoder LLM)."""
