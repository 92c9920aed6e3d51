// Minimal chat client: keeps the conversation in memory, posts it to /api/chat and renders the
// Server-Sent Events stream as it arrives. No dependencies.
"use strict";

const $ = (id) => document.getElementById(id);
const transcript = $("messages");
const knobs = ["temperature", "top_p", "top_k", "max_new_tokens"];
let messages = [];
let controller = null;

function escapeHtml(text) {
  return text.replace(/[&<>]/g, (c) => ({ "&": "&amp;", "<": "&lt;", ">": "&gt;" }[c]));
}

// Tiny markdown subset: fenced code, inline code, bold.
function render(text) {
  const parts = escapeHtml(text).split(/```/);
  return parts
    .map((part, i) =>
      i % 2 === 1
        ? `<pre>${part.replace(/^\w*\n/, "")}</pre>`
        : part.replace(/`([^`]+)`/g, "<code>$1</code>").replace(/\*\*([^*]+)\*\*/g, "<b>$1</b>")
    )
    .join("");
}

function addTurn(role, text) {
  const node = document.createElement("div");
  node.className = `turn ${role}`;
  node.innerHTML = render(text);
  transcript.appendChild(node);
  transcript.scrollTop = transcript.scrollHeight;
  return node;
}

function setBusy(busy) {
  $("send").hidden = busy;
  $("stop").hidden = !busy;
}

async function loadInfo() {
  try {
    const info = await (await fetch("/api/info")).json();
    const m = info.model;
    $("model-chip").textContent =
      `${(m.parameters / 1e6).toFixed(0)}M · ${m.layers}L · ctx ${m.context_length} · ${m.dtype}`;
    for (const key of knobs) {
      $(key).value = info.defaults[key];
      $(`${key}-value`).textContent = info.defaults[key];
    }
  } catch (error) {
    $("model-chip").textContent = "offline";
  }
}

async function send(text) {
  messages.push({ role: "user", content: text });
  addTurn("user", text);
  const node = addTurn("assistant streaming", "");
  const body = { messages };
  for (const key of knobs) body[key] = Number($(key).value);
  if ($("seed").value !== "") body.seed = Number($("seed").value);
  controller = new AbortController();
  setBusy(true);
  let reply = "";
  let pieces = 0;
  const started = performance.now();
  try {
    const response = await fetch("/api/chat", {
      method: "POST",
      headers: { "Content-Type": "application/json" },
      body: JSON.stringify(body),
      signal: controller.signal,
    });
    if (!response.ok) throw new Error((await response.json()).error || response.statusText);
    const reader = response.body.getReader();
    const decoder = new TextDecoder();
    let buffer = "";
    for (;;) {
      const { value, done } = await reader.read();
      if (done) break;
      buffer += decoder.decode(value, { stream: true });
      let cut;
      while ((cut = buffer.indexOf("\n\n")) >= 0) {
        const frame = buffer.slice(0, cut);
        buffer = buffer.slice(cut + 2);
        if (!frame.startsWith("data: ")) continue;
        const event = JSON.parse(frame.slice(6));
        if (event.error) throw new Error(event.error);
        if (event.delta) {
          reply += event.delta;
          pieces += 1;
          node.innerHTML = render(reply);
          transcript.scrollTop = transcript.scrollHeight;
          const seconds = (performance.now() - started) / 1000;
          $("speed").hidden = false;
          $("speed").textContent = `${(pieces / Math.max(seconds, 1e-3)).toFixed(1)} tok/s`;
        }
      }
    }
    messages.push({ role: "assistant", content: reply });
  } catch (error) {
    if (error.name === "AbortError") {
      if (reply) messages.push({ role: "assistant", content: reply });
      else messages.pop();
    } else {
      messages.pop();
      addTurn("error", String(error.message || error));
    }
  } finally {
    node.classList.remove("streaming");
    controller = null;
    setBusy(false);
  }
}

$("composer-form").addEventListener("submit", (event) => {
  event.preventDefault();
  const text = $("prompt").value.trim();
  if (!text || controller) return;
  $("prompt").value = "";
  send(text);
});
$("prompt").addEventListener("keydown", (event) => {
  if (event.key === "Enter" && !event.shiftKey) {
    event.preventDefault();
    $("composer-form").requestSubmit();
  }
});
$("stop").addEventListener("click", () => controller && controller.abort());
$("new-chat").addEventListener("click", () => {
  if (controller) controller.abort();
  messages = [];
  transcript.innerHTML = "";
});
$("settings-toggle").addEventListener("click", () => {
  $("settings").hidden = !$("settings").hidden;
});
for (const key of knobs) {
  $(key).addEventListener("input", () => ($(`${key}-value`).textContent = $(key).value));
}
loadInfo();
