class ModelSummary:
    """Parameter counts only; enough for ``ohara.utils.info.model_summary``."""

    def __init__(self, model, *args, **kwargs):
        params = list(model.parameters())
        self.total_parameters = sum(p.numel() for p in params)
        self.trainable_parameters = sum(p.numel() for p in params if p.requires_grad)

    def __str__(self):
        return f"total={self.total_parameters} trainable={self.trainable_parameters}"
