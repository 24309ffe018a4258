"""B200-native K-FAC curvature path behind the PyTorch-SSO API."""
