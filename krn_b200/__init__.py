"""B200-native implementation of the dense-contraction path of the krn kernel language."""
