"""CPU oracle package (test infrastructure only; never imported by llmini_b200)."""
