"""B200-native trace post-processing for libkineto: CUPTI activity records -> Chrome-trace JSON."""
