"""TEST INFRASTRUCTURE ONLY: the CPU oracle (C restatement + doors to the compiled reference)."""
