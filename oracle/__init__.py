"""CPU checkers for the fused pre-processing path. TEST INFRASTRUCTURE ONLY: the product package never imports this."""
