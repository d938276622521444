from fastdms_b200.engine.llm_engine import LLMEngine


class LLM(LLMEngine):
    """`LLM(model, **config).generate(prompts, sampling_params)` as in the reference's `fastdms.LLM`.
    Prompts are strings (the model directory must then hold tokenizer files) or lists of token ids."""
