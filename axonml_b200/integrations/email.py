"""Transactional e-mail through the Resend HTTP API (crates/axonml-server/src/email.rs:37-370):
verification link, administrator notification of a sign-up, approval request, welcome message.
Without an API key the service reports ``is_configured() == False`` and the server approves
accounts at once instead of mailing."""
from __future__ import annotations

import html
import json
import urllib.error
import urllib.request


class EmailError(RuntimeError):
    pass


class EmailService:
    def __init__(self, api_key: str | None = None, sender: str = "AxonML <noreply@axonml.local>",
                 base_url: str = "https://api.resend.com", timeout: float = 10.0):
        self.api_key, self.sender, self.base_url, self.timeout = api_key, sender, base_url.rstrip("/"), timeout
        self.sent: list[dict] = []          # ids and recipients of what went out (for the admin page and tests)

    def is_configured(self) -> bool:
        return bool(self.api_key)

    def _send(self, to: str, subject: str, body_html: str) -> str:
        if not self.is_configured():
            raise EmailError("no e-mail API key is configured")
        payload = {"from": self.sender, "to": [to], "subject": subject, "html": body_html}
        req = urllib.request.Request(self.base_url + "/emails", data=json.dumps(payload).encode(), method="POST")
        req.add_header("Authorization", f"Bearer {self.api_key}")
        req.add_header("Content-Type", "application/json")
        try:
            with urllib.request.urlopen(req, timeout=self.timeout) as r:
                out = json.loads(r.read() or b"{}")
        except urllib.error.HTTPError as e:
            raise EmailError(f"the e-mail service answered {e.code}") from e
        except (urllib.error.URLError, OSError) as e:
            raise EmailError(f"the e-mail service is unreachable: {e}") from e
        self.sent.append({"id": out.get("id"), "to": to, "subject": subject})
        return str(out.get("id", ""))

    @staticmethod
    def _page(title: str, paragraphs: list[str], link: str | None = None, link_text: str = "") -> str:
        parts = [f"<h2>{html.escape(title)}</h2>"] + [f"<p>{html.escape(p)}</p>" for p in paragraphs]
        if link:
            parts.append(f'<p><a href="{html.escape(link, quote=True)}">{html.escape(link_text or link)}</a></p>')
        return "<div style=\"font-family:sans-serif\">" + "".join(parts) + "</div>"

    def send_verification_email(self, to: str, name: str, verify_url: str) -> str:
        return self._send(to, "Verify your AxonML e-mail address",
                          self._page(f"Welcome, {name}", ["Confirm this address to finish creating your account.",
                                                         "The link is valid for 24 hours."], verify_url, "Verify e-mail"))

    def send_admin_signup_notification(self, admin: str, user_email: str, user_name: str) -> str:
        return self._send(admin, f"New AxonML sign-up: {user_email}",
                          self._page("New sign-up", [f"{user_name} <{user_email}> registered and is verifying the address."]))

    def send_admin_approval_request(self, admin: str, user_email: str, user_name: str, approve_url: str) -> str:
        return self._send(admin, f"Approve AxonML account: {user_email}",
                          self._page("Approval requested", [f"{user_name} <{user_email}> verified the address and waits for approval."],
                                     approve_url, "Approve account"))

    def send_welcome_email(self, to: str, name: str, login_url: str) -> str:
        return self._send(to, "Your AxonML account is ready",
                          self._page(f"Hello {name}", ["Your account has been approved."], login_url, "Sign in"))
