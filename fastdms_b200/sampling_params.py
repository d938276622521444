from dataclasses import dataclass


@dataclass(slots=True)
class SamplingParams:
    """Per-request sampling options (same fields as the reference's SamplingParams)."""
    temperature: float = 1.0
    max_tokens: int = 64
    ignore_eos: bool = False

    def __post_init__(self):
        assert self.temperature >= 0.0, "temperature must be non-negative"
