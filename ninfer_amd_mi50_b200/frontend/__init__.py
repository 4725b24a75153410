"""Text in and out: tokenizer and chat template (outside the token-to-token path)."""
