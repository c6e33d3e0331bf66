"""Import stand-in: the reference imports peft only in its `download-weights` PEFT-merge path."""


class _Unavailable:
    @classmethod
    def from_pretrained(cls, *a, **k):
        raise RuntimeError("peft is not installed")


AutoPeftModelForCausalLM = _Unavailable
AutoPeftModelForSeq2SeqLM = _Unavailable
LoraConfig = _Unavailable
