"""B200-native inference engine for the dense Llama decoder."""
