"""Stand-in for ``optimum.bettertransformer`` (not installed).  ``BetterTransformer.transform`` swapped
GPT-2's eager attention for ``torch.nn.functional.scaled_dot_product_attention``; current
``transformers`` already selects that SDPA path natively, so the transform is the identity here."""


class BetterTransformer:
    @staticmethod
    def transform(model, **kwargs):
        return model
