"""The engine: step function, scheduler, generation and trace replay."""
