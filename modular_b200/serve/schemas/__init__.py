"""Request / response schemas of the HTTP APIs."""
