"""CPU oracle of the speculative-decoding step.  Test infrastructure only."""
