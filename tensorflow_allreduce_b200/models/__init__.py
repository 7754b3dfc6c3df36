"""Models of the benchmark configurations (plain torch.nn): DeepSpeech2-style, GPT-2, ResNet-50."""
